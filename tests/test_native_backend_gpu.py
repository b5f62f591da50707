"""Native sm_100a executor against the fp32 CPU interpreter on synthetic models."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _feed(plan, feeds):
    for k, v in feeds.items():
        dst = plan.inputs[k]
        t = torch.from_numpy(v).cuda()
        if dst.nhwc:
            dst.t.copy_(t.permute(0, 2, 3, 1))
        else:
            dst.t.copy_(t)


def test_resnet_like_matches_interpreter():
    from fastdeploy_b200.importer.onnx_format import load_onnx
    from fastdeploy_b200.ir.interp import Interpreter
    from fastdeploy_b200.models.resnet import resnet18_like_onnx
    from fastdeploy_b200.runtime.native_backend import build_plan
    g = load_onnx(resnet18_like_onnx())
    x = np.random.RandomState(0).rand(4, 3, 64, 64).astype(np.float32)
    ref = Interpreter(g).run({"input": x})["output"]
    plan = build_plan(g, {"input": [4, 3, 64, 64]}, "cuda:0")
    _feed(plan, {"input": x})
    plan.run()
    torch.cuda.synchronize()
    plan.status.check()
    out = plan.outputs["output"].logical().float().cpu()
    assert out.shape == ref.shape
    assert (out - ref).abs().max().item() < 3e-2 * ref.abs().max().item() + 1e-3
    assert plan.native_kernel_launches >= 18
    # captured replay gives the same answer
    plan.capture()
    plan.run()
    torch.cuda.synchronize()
    out2 = plan.outputs["output"].logical().float().cpu()
    assert torch.equal(out, out2)


@pytest.mark.parametrize("with_nms", [False, True])
def test_ppyoloe_tiny_matches_interpreter(with_nms):
    from fastdeploy_b200.importer.paddle_import import load_paddle
    from fastdeploy_b200.ir.interp import Interpreter
    from fastdeploy_b200.models.ppyoloe import build_ppyoloe
    from fastdeploy_b200.runtime.native_backend import build_plan
    net = build_ppyoloe("tiny", image=128, num_classes=8, with_nms=with_nms, score_threshold=0.005)
    m, p = net.serialize()
    g = load_paddle(m, p)
    rng = np.random.RandomState(1)
    x = rng.rand(2, 3, 128, 128).astype(np.float32)
    sf = np.array([[1.0, 1.0], [0.5, 0.75]], np.float32)
    ref = Interpreter(g).run({"image": x, "scale_factor": sf})
    plan = build_plan(g, {"image": [2, 3, 128, 128], "scale_factor": [2, 2]}, "cuda:0")
    _feed(plan, {"image": x, "scale_factor": sf})
    plan.run()
    torch.cuda.synchronize()
    plan.status.check()
    names = g.output_names()
    if not with_nms:
        boxes = plan.outputs[names[0]].logical().float().cpu()
        scores = plan.outputs[names[1]].logical().float().cpu()
        assert (boxes - ref[names[0]]).abs().max().item() < 1.0          # pixels, fp16 network
        assert (scores - ref[names[1]]).abs().max().item() < 2e-2
    else:
        num = plan.outputs[names[1]].t.cpu().numpy()
        ref_num = ref[names[1]].numpy()
        # fp16 scores may move a few candidates across the threshold
        assert np.all(np.abs(num - ref_num) <= 5)
        out = plan.outputs[names[0]].t.cpu().numpy().reshape(2, -1, 6)
        ref_out = ref[names[0]].numpy()
        pos = 0
        for i in range(2):
            got = out[i, :num[i]]
            want = ref_out[pos:pos + ref_num[i]]
            pos += ref_num[i]
            k = min(len(got), len(want), 10)
            # the strongest detections agree
            assert np.allclose(np.sort(got[:, 1])[::-1][:k], np.sort(want[:, 1])[::-1][:k], atol=2e-2)


@pytest.mark.parametrize("task", ["seq_cls", "uie"])
def test_ernie_tiny_matches_interpreter(task):
    from fastdeploy_b200.importer.paddle_import import load_paddle
    from fastdeploy_b200.ir.interp import Interpreter
    from fastdeploy_b200.models.ernie import build_ernie
    from fastdeploy_b200.runtime.native_backend import build_plan
    g = load_paddle(*build_ernie("tiny", task).serialize())
    B, S = 3, 24
    rng = np.random.RandomState(0)
    ids = rng.randint(1, 1000, (B, S)).astype(np.int64)
    ids[1, 15:] = 0
    feeds = {"input_ids": ids, "token_type_ids": rng.randint(0, 2, (B, S)).astype(np.int64)}
    if task == "uie":
        feeds["pos_ids"] = np.tile(np.arange(S), (B, 1)).astype(np.int64)
        feeds["att_mask"] = (ids != 0).astype(np.int64)
    ref = Interpreter(g).run(feeds)
    plan = build_plan(g, {k: list(v.shape) for k, v in feeds.items()}, "cuda:0", dtype=torch.bfloat16)
    _feed(plan, feeds)
    plan.run()
    torch.cuda.synchronize()
    plan.status.check()
    for k, r in ref.items():
        out = plan.outputs[k].logical().float().cpu()
        assert out.shape == r.shape
        assert (out - r).abs().max().item() < 3e-2
    names = [s.name for s in plan.steps]
    assert any(n.startswith("attn_qk") or n == "attention" for n in names) and any(n == "layernorm" for n in names)


def test_plan_trace_is_a_chrome_trace_document(tmp_path):
    import json
    import fastdeploy_b200 as fd
    from fastdeploy_b200.models.resnet import resnet18_like_onnx
    path = tmp_path / "m.onnx"
    path.write_bytes(resnet18_like_onnx())
    opt = fd.RuntimeOption()
    opt.set_model_path(str(path), "", fd.ModelFormat.ONNX)
    opt.use_gpu(0)
    rt = fd.Runtime(opt)
    out = tmp_path / "trace.json"
    doc = rt.export_trace({"input": [4, 3, 64, 64]}, str(out))
    loaded = json.loads(out.read_text())
    assert loaded["otherData"]["steps"] == len(doc["traceEvents"]) >= 18
    ev = loaded["traceEvents"]
    assert all(e["ph"] == "X" and e["dur"] > 0 and e["cat"] == "native" for e in ev)
    assert all(ev[i + 1]["ts"] >= ev[i]["ts"] for i in range(len(ev) - 1))
    assert any(e["name"].startswith("conv") for e in ev)


def test_activation_arena_reuses_buffers_without_changing_results():
    """Static memory plan: with buffer reuse the plan needs less activation memory than the sum of its buffers and
    returns bit-identical outputs, eagerly and as a CUDA graph, run after run."""
    from fastdeploy_b200.importer.paddle_import import load_paddle
    from fastdeploy_b200.models.ppyoloe import build_ppyoloe
    from fastdeploy_b200.runtime.native_backend import build_plan
    net = build_ppyoloe("s", image=320, num_classes=16, with_nms=False)
    m, p = net.serialize()
    g = load_paddle(m, p)
    rng = np.random.RandomState(2)
    shapes = {"image": [4, 3, 320, 320], "scale_factor": [4, 2]}
    feeds = [{"image": rng.rand(4, 3, 320, 320).astype(np.float32), "scale_factor": np.ones((4, 2), np.float32)}
             for _ in range(2)]
    plain = build_plan(g, shapes, "cuda:0", reuse_buffers=False)
    pooled = build_plan(g, shapes, "cuda:0", reuse_buffers=True)
    assert "memory" not in plain.extra
    mem = pooled.extra["memory"]
    assert 0 < mem["peak_live_bytes"] <= mem["arena_bytes"] < 0.7 * mem["requested_bytes"], mem
    names = g.output_names()
    pooled.capture()
    for rep in range(3):
        f = feeds[rep % 2]
        outs = []
        for plan in (plain, pooled):
            _feed(plan, f)
            plan.run()
            torch.cuda.synchronize()
            plan.status.check()
            outs.append([plan.outputs[n].logical().float().cpu().clone() for n in names])
        for a, b in zip(*outs):
            assert torch.equal(a, b), rep


def test_batch_buckets_pad_to_a_built_plan_and_cut_the_outputs_back(tmp_path):
    """Ragged batches run in the smallest bucket plan: one plan for batches 3 and 4, the same answers as exact plans."""
    import fastdeploy_b200 as fd
    from fastdeploy_b200.models.ppyoloe import write_ppyoloe
    paths = write_ppyoloe(str(tmp_path), "tiny", image=128, num_classes=8, score_threshold=0.005)
    rng = np.random.RandomState(4)

    def runtime(buckets):
        opt = fd.RuntimeOption()
        opt.use_gpu(0)
        opt.set_model_path(paths["model"], paths["params"])
        if buckets:
            opt.set_batch_buckets(buckets)
        return fd.Runtime(opt)
    bucketed = runtime([1, 2, 4, 8])
    names = [vi.name for vi in bucketed.graph.outputs]
    for n in (3, 4, 1, 3):
        img = rng.rand(4, 3, 128, 128).astype(np.float32)
        part = bucketed.infer({"image": img[:n], "scale_factor": np.ones((n, 2), np.float32)})
        if n == 1:
            assert part[1].shape == (1,)
            continue
        # the same images as the head of a full bucket: every image's detections are its own
        full = bucketed.infer({"image": img, "scale_factor": np.ones((4, 2), np.float32)})
        counts = part[1].reshape(-1)
        assert counts.shape == (n,) and np.array_equal(counts, full[1].reshape(-1)[:n]), names
        assert part[0].shape[0] == counts.sum() and np.array_equal(part[0], full[0][:counts.sum()])
    assert sorted(dict(k)["image"][0] for k in bucketed._plans) == [1, 4]
