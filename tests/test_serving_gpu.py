"""serving.Scheduler driving real models on every visible GPU from one process: one worker thread, stream and model
per GPU, single-frame requests grouped by the native batching core."""
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_scheduler_serves_detection_requests_on_all_visible_gpus(tmp_path):
    import fastdeploy_b200 as fd
    from fastdeploy_b200.models.ppyoloe import write_ppyoloe
    from fastdeploy_b200.serving import Scheduler
    n_gpu = torch.cuda.device_count()
    d = str(tmp_path / "pp")
    # 640 x 640 puts the NMS kernel above the default 48 KB of dynamic shared memory: the opt-in must reach every GPU
    write_ppyoloe(d, "tiny", image=640, num_classes=8, seed=0, score_threshold=0.005, nms_threshold=0.6, nms_top_k=200,
                  keep_top_k=20)

    def make(i):
        opt = fd.RuntimeOption()
        opt.use_gpu(i)
        opt.enable_trt_fp16()
        return fd.vision.detection.PPYOLOE(os.path.join(d, "model.pdmodel"), os.path.join(d, "model.pdiparams"),
                                           os.path.join(d, "infer_cfg.yml"), runtime_option=opt)
    rng = np.random.default_rng(0)
    frames = [rng.integers(0, 256, (96, 160, 3), dtype=np.uint8) for _ in range(6)]
    direct = make(0)
    batch = 4
    # the oracle runs the same batch compositions through the model directly (same plan shape as the workers use)
    want = {k: direct.batch_predict([frames[(k + j) % len(frames)] for j in range(batch)]) for k in range(len(frames))}
    sched = Scheduler(make, lambda m, xs: m.predict_async(xs), num_workers=n_gpu, max_batch_size=batch,
                      max_queue_delay_us=2000, pipeline_depth=2)
    try:
        futs = []
        for k in range(10 * n_gpu):                     # bursts that stay together, spread over the workers
            futs.append(sched.submit_many([frames[(k + j) % len(frames)] for j in range(batch)], together=True))
        singles = [sched.submit(frames[i]) for i in range(len(frames))]
        for k, fs in enumerate(futs):
            for j, f in enumerate(fs):
                got = f.result(60)
                ref = want[k % len(frames)][j]
                assert got.label_ids == ref.label_ids
                assert np.allclose(got.boxes, ref.boxes, atol=1e-3) and np.allclose(got.scores, ref.scores, atol=1e-5)
        for f in singles:                               # lone requests are batched with whatever else is queued
            r = f.result(60)
            assert len(r.boxes) == len(r.scores) == len(r.label_ids) and len(r.boxes) <= 20
        st = sched.stats()
        workers = st["workers"]
        assert len(workers) == n_gpu and sum(w["requests"] for w in workers) == 10 * n_gpu * batch + len(frames)
        assert all(w["requests"] > 0 and w["failed"] == 0 for w in workers)         # every GPU took part
        assert max(w["avg_batch_size"] for w in workers) > 1.5
        text = sched.metrics_text()
        assert "requests_total" in text or "fdb_" in text
    finally:
        sched.close()
