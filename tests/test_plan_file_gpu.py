"""Exported plans replayed by the C++ runner (a process without Python) give the bytes the Python plan gives."""
import os
import subprocess

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _roundtrip(plan, feeds, tmp_path, tag):
    """Runs ``plan`` in Python on ``feeds`` (name -> tensor in the plan input's own layout), exports it, replays it
    with the command-line runner on the same bytes and compares every output bit for bit."""
    from fastdeploy_b200._native import KERNEL_LIB
    from fastdeploy_b200._native import build
    from fastdeploy_b200._native.build import RUNNER_TOOL
    from fastdeploy_b200.runtime.plan_file import export_plan
    if not os.path.exists(RUNNER_TOOL):
        build.build_runner()
    path = str(tmp_path / f"{tag}.fdplan")
    info = export_plan(plan, path)
    assert info["ops"] == len(plan.steps) and info["constant_bytes"] > 0
    for name, t in feeds.items():
        plan.inputs[name].t.copy_(t)
    plan.run()
    torch.cuda.synchronize()
    plan.status.check()
    want = {n: v.t.contiguous().cpu() for n, v in plan.outputs.items()}
    cmd = [RUNNER_TOOL, path, KERNEL_LIB]
    for k, name in enumerate(info["inputs"]):
        f = str(tmp_path / f"{tag}_in{k}.bin")
        feeds[name].contiguous().cpu().numpy().tofile(f) if feeds[name].dtype != torch.bfloat16 else \
            feeds[name].contiguous().cpu().view(torch.int16).numpy().tofile(f)
        cmd += ["--in", str(k), f]
    outs = []
    for k, name in enumerate(info["outputs"]):
        f = str(tmp_path / f"{tag}_out{k}.bin")
        outs.append((name, f))
        cmd += ["--out", str(k), f]
    cmd += ["--iters", "5"]
    run = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=600)
    assert run.returncode == 0, run.stdout[-3000:]
    assert "ms_per_run" in run.stdout
    for name, f in outs:
        got = np.fromfile(f, dtype=np.uint8)
        ref = want[name].view(torch.uint8).numpy().reshape(-1) if want[name].numel() else np.zeros(0, np.uint8)
        assert got.size == ref.size, (name, got.size, ref.size)
        assert np.array_equal(got, ref), name
    return info


def test_convolutional_plan_replays_without_python(tmp_path):
    from fastdeploy_b200.importer.onnx_format import load_onnx
    from fastdeploy_b200.models.resnet import resnet18_like_onnx
    from fastdeploy_b200.runtime.native_backend import build_plan
    g = load_onnx(resnet18_like_onnx())
    plan = build_plan(g, {"input": [4, 3, 64, 64]}, "cuda:0")
    x = torch.rand(4, 64, 64, 3, device="cuda").to(plan.inputs["input"].t.dtype)       # the plan input is NHWC
    info = _roundtrip(plan, {"input": x}, tmp_path, "resnet")
    assert info["inputs"] == ["input"]


def test_detector_plan_with_nms_replays_without_python(tmp_path):
    from fastdeploy_b200.importer.paddle_import import load_paddle
    from fastdeploy_b200.models.ppyoloe import build_ppyoloe
    from fastdeploy_b200.runtime.native_backend import build_plan
    net = build_ppyoloe("tiny", image=128, num_classes=8, with_nms=True, score_threshold=0.005)
    m, p = net.serialize()
    plan = build_plan(load_paddle(m, p), {"image": [2, 3, 128, 128], "scale_factor": [2, 2]}, "cuda:0")
    feeds = {"image": torch.rand(2, 128, 128, 3, device="cuda").to(plan.inputs["image"].t.dtype),
             "scale_factor": torch.ones(2, 2, device="cuda")}
    _roundtrip(plan, feeds, tmp_path, "ppyoloe")


def test_encoder_plan_with_pointer_tables_replays_without_python(tmp_path):
    import fastdeploy_b200 as fd
    from fastdeploy_b200.models.ernie import write_ernie
    write_ernie(str(tmp_path), "tiny", "seq_cls", seed=1, vocab=False)
    opt = fd.RuntimeOption()
    opt.use_gpu(0)
    opt.set_model_path(str(tmp_path / "model.pdmodel"), str(tmp_path / "model.pdiparams"))
    rt = fd.Runtime(opt)
    plan = rt.plan_for_shapes({"input_ids": [3, 32], "token_type_ids": [3, 32]})
    ids = torch.randint(1, 1000, (3, 32), device="cuda")
    ids[1, 20:] = 0
    info = _roundtrip(plan, {"input_ids": ids, "token_type_ids": torch.zeros_like(ids)}, tmp_path, "ernie")
    assert info["pointer_tables"] == 2
