"""Padding-free encoder plans on the GPU: same logits as the padded plan, one CUDA graph for every batch composition."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _runtime(fd, d, precision):
    opt = fd.RuntimeOption()
    opt.use_gpu(0)
    opt.native_option.precision = precision
    opt.set_model_path(str(d / "model.pdmodel"), str(d / "model.pdiparams"))
    return fd.Runtime(opt)


@pytest.mark.parametrize("task", ["seq_cls", "uie"])
def test_packed_plan_matches_padded_plan(tmp_path, task):
    import fastdeploy_b200 as fd
    from fastdeploy_b200.models.ernie import write_ernie
    from fastdeploy_b200.text.packed import PackedEncoder
    write_ernie(str(tmp_path), "tiny", task, seed=1, vocab=False)
    rt = _runtime(fd, tmp_path, "fp16")
    names = [vi.name for vi in rt.graph.inputs]
    enc = PackedEncoder(rt, max_tokens=512, max_seqs=8, max_len=128, token_buckets=[256])
    rng = np.random.default_rng(3)
    for lens in ([5, 64, 17, 100, 1], [128, 90, 100], [31, 32, 33, 8, 8, 8, 100, 2]):
        seqs = []
        for n in lens:
            s = [rng.integers(1, 1000, n), rng.integers(0, 2, n)]
            if task == "uie":
                s += [np.arange(n), np.ones(n, np.int64)]
            seqs.append(tuple(s))
        outs = enc.infer(seqs)
        feeds = {n: np.zeros((len(lens), 128), np.int64) for n in names}
        for i, s in enumerate(seqs):
            for n, a in zip(names, s):
                feeds[n][i, :len(a)] = a
        ref = rt.infer(feeds)
        if task == "seq_cls":
            assert outs[0].shape == ref[0].shape
            assert np.abs(outs[0] - ref[0]).max() < 2e-3, lens
        else:
            for k in range(2):
                for i, n in enumerate(lens):
                    assert np.abs(outs[k][i] - ref[k][i, :n]).max() < 5e-3, (lens, k, i)
    assert sorted(enc._buckets) == [256, 512]
    for bk in enc._buckets.values():
        assert [s.name for s in bk.plan.steps if s.native is None] == []
        assert bk.plan.graph is not None                       # replayed as one CUDA graph
