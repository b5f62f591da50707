"""precision = "fp8" through the public Runtime: linear layers on e4m3 operands, dynamic per-row activation
quantisation by default, static ranges from a QDQ export or a calibration file."""
import json
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _write(tmp_path, b):
    m, p = b.serialize()
    mf, pf = str(tmp_path / "m.pdmodel"), str(tmp_path / "m.pdiparams")
    open(mf, "wb").write(m)
    open(pf, "wb").write(p)
    return mf, pf


def test_quantize_rows_kernel_matches_reference():
    from fastdeploy_b200.ops import nhwc as K
    g = torch.Generator().manual_seed(0)
    x = (torch.randn(37, 200, generator=g) * torch.rand(37, 1, generator=g) * 5).cuda().bfloat16()
    buf = torch.zeros(37, 208, dtype=torch.bfloat16, device="cuda")
    buf[:, :200] = x
    q = torch.full((37, 256), 1.0, device="cuda").to(torch.float8_e4m3fn)
    s = torch.zeros(37, device="cuda")
    K.quantize_rows_e4m3_op(buf, q, s, rows=37, c=200, x_ld=208, y_ld=256, c_padded=256).launch()
    torch.cuda.synchronize()
    amax = x.float().abs().amax(1)
    torch.testing.assert_close(s, amax / 448.0, rtol=1e-6, atol=0)
    ref = (x.float() * (448.0 / amax)[:, None]).to(torch.float8_e4m3fn).float()
    got = q[:, :200].float()
    # identical up to rounding ties of the scaled value: at most one e4m3 step (2^-3 relative), and rare
    assert float(((got - ref).abs() <= 0.126 * ref.abs() + 2.0 ** -9).float().mean()) == 1.0
    assert float((got == ref).float().mean()) > 0.98, float((got == ref).float().mean())
    assert float(q[:, 200:].float().abs().max()) == 0.0


@pytest.mark.parametrize("static", [False, True])
def test_ernie_fp8_logits_close_to_fp32(tmp_path, static):
    import fastdeploy_b200 as fd
    from fastdeploy_b200.ir.interp import Interpreter
    from fastdeploy_b200.models.ernie import write_ernie
    from fastdeploy_b200.tools import calibrate
    d = str(tmp_path / "ernie")
    write_ernie(d, "tiny", "seq_cls", seed=0, vocab=False)
    rng = np.random.RandomState(0)
    ids = rng.randint(1, 100, size=(8, 32)).astype(np.int64)
    ids[2, 20:] = 0
    feeds = {"input_ids": ids, "token_type_ids": np.zeros((8, 32), np.int64)}
    opt = fd.RuntimeOption()
    opt.set_model_path(os.path.join(d, "model.pdmodel"), os.path.join(d, "model.pdiparams"))
    cpu = fd.Runtime(opt)
    feeds = {vi.name: feeds[vi.name] for vi in cpu.graph.inputs}
    ref = np.asarray(cpu.infer(feeds)[0], np.float32)
    if static:
        # ranges of every linear layer's input from the calibration tool, keyed by tensor name
        from fastdeploy_b200.ir import passes
        g = passes.optimize(cpu.graph, {k: list(v.shape) for k, v in feeds.items()})
        scales = calibrate(g, [feeds])
        with open(os.path.join(d, "quant_scales.json"), "w") as f:
            json.dump({"format": "e4m3", "layers": scales}, f)
    gopt = fd.RuntimeOption()
    gopt.set_model_path(os.path.join(d, "model.pdmodel"), os.path.join(d, "model.pdiparams"))
    gopt.use_gpu(0)
    gopt.enable_fp8()
    rt = fd.Runtime(gopt)
    out = np.asarray(rt.infer(feeds)[0], np.float32)
    plan = rt.plan_for_shapes({k: list(v.shape) for k, v in feeds.items()})
    names = [s.name for s in plan.steps]
    assert plan.extra["fp8_gemms"] >= 4 and any(n.startswith("gemm_fp8") for n in names)
    assert [s.name for s in plan.steps if s.native is None] == []
    if static:
        assert "quantize_e4m3" in names and rt.act_scales
    else:
        assert "quantize_rows_e4m3" in names
    assert out.shape == ref.shape
    assert (out.argmax(1) == ref.argmax(1)).mean() >= 0.75
    assert np.abs(out - ref).max() <= 0.08 * np.abs(ref).max() + 0.02


def test_qdq_model_runs_fp8_with_its_own_ranges(tmp_path):
    import fastdeploy_b200 as fd
    from test_importer_ops_extra import _qdq_mlp
    b, _ = _qdq_mlp()
    mf, pf = _write(tmp_path, b)
    x = np.random.RandomState(1).uniform(-2.5, 2.5, (128, 64)).astype(np.float32)
    copt = fd.RuntimeOption()
    copt.set_model_path(mf, pf)
    ref = np.asarray(fd.Runtime(copt).infer({"x": x})[0], np.float32)       # fake-quantised int8 forward on the CPU
    gopt = fd.RuntimeOption()
    gopt.set_model_path(mf, pf)
    gopt.use_gpu(0)
    gopt.enable_fp8()
    rt = fd.Runtime(gopt)
    out = np.asarray(rt.infer({"x": x})[0], np.float32)
    plan = rt.plan_for_shapes({"x": [128, 64]})
    names = [s.name for s in plan.steps]
    assert names.count("quantize_e4m3") == 2 and plan.extra["fp8_gemms"] == 2      # static ranges from the QDQ pairs
    err = np.abs(out - ref)
    assert err.max() <= 0.06 * np.abs(ref).max() + 0.02, err.max()
    assert np.corrcoef(out.ravel(), ref.ravel())[0, 1] > 0.998
