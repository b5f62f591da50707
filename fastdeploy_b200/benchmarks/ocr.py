"""PP-OCRv3 (detector + angle classifier + recogniser with a 6625-character vocabulary), fp16, pages of 960 x 960
uint8, 20 - 60 text boxes per page, data-parallel over pages. The reference's drivers are
benchmark/cpp/benchmark_ppocr_{det,cls,rec}.cc (one stage each) and the pipeline in
fastdeploy/vision/ocr/ppocr/ppocr_v2.cc:108-175.

A random-init detector finds no text, so the crops that the classifier and the recogniser read come from the
synthetic page layout (the boxes the page was drawn with); the detector and the device DB post-processing still
run on every page, on the detector's own output, inside the timed region."""
from __future__ import annotations

import os
import tempfile

from .common import ClockSampler, Context, median, physical_gpu_index, spread


def make_pages(rng, n: int, hw: int):
    """White pages with dark text-line rectangles: 20 - 60 boxes per page, heights 18 - 40 px, aspect 2 - 16, a few of
    them slightly rotated. Returns the uint8 pages and the boxes (clockwise from the top-left corner)."""
    import numpy as np
    pages = np.full((n, hw, hw, 3), 235, np.uint8)
    all_boxes = []
    for p in range(n):
        boxes = []
        for _ in range(int(rng.integers(20, 61))):
            h = int(rng.integers(18, 41))
            w = int(min(h * rng.uniform(2.0, 16.0), hw - 40))
            x0 = int(rng.integers(10, hw - w - 10))
            y0 = int(rng.integers(10, hw - h - 10))
            ang = float(rng.uniform(-0.05, 0.05)) if rng.random() < 0.3 else 0.0
            c, s = np.cos(ang), np.sin(ang)
            cx, cy = x0 + w / 2, y0 + h / 2
            pts = []
            for dx, dy in ((-w / 2, -h / 2), (w / 2, -h / 2), (w / 2, h / 2), (-w / 2, h / 2)):
                pts += [int(np.clip(round(cx + dx * c - dy * s), 0, hw - 1)), int(np.clip(round(cy + dx * s + dy * c), 0, hw - 1))]
            boxes.append(pts)
            pages[p, y0:y0 + h, x0:x0 + w] = rng.integers(0, 120, (h, w, 3), dtype=np.uint8)
        all_boxes.append(boxes)
    return pages, all_boxes


def run(ctx: Context, args) -> dict:
    import numpy as np
    torch = ctx.torch
    import fastdeploy_b200 as fd
    from fastdeploy_b200.models import ppocr
    from fastdeploy_b200.vision.ocr.device_pipeline import DeviceOCR
    fd.set_logger(False, True)
    dev = ctx.dev
    model_dir = args.model_dir or os.path.join(tempfile.gettempdir(), "fdb200_ppocrv3")
    if ctx.rank == 0 and not os.path.exists(os.path.join(model_dir, "rec.pdiparams")):
        ppocr.write_ppocr(model_dir, seed=0, vocab=6625)
    ctx.barrier()

    def option():
        o = fd.RuntimeOption()
        o.use_gpu(ctx.local_rank)
        o.enable_trt_fp16()
        return o
    j = lambda f: os.path.join(model_dir, f)
    det = fd.vision.ocr.DBDetector(j("det.pdmodel"), j("det.pdiparams"), runtime_option=option())
    cls = fd.vision.ocr.Classifier(j("cls.pdmodel"), j("cls.pdiparams"), runtime_option=option())
    rec = fd.vision.ocr.Recognizer(j("rec.pdmodel"), j("rec.pdiparams"), j("ppocr_keys_v1.txt"), runtime_option=option())
    ocr = DeviceOCR(det, cls, rec)
    B, HW = args.batch or 8, 960
    rng = np.random.default_rng(7 + ctx.rank)
    sets = []
    for _ in range(3):
        pages, boxes = make_pages(rng, B, HW)
        host = torch.from_numpy(pages).pin_memory()
        sets.append((host, host.to(dev), boxes))
    n_boxes = sum(len(b) for _, _, bl in sets for b in bl) / 3
    sampler = ClockSampler(physical_gpu_index(ctx.local_rank))
    sampler.start()
    ocr.warm_up((HW, HW), B)
    flush = torch.empty(192 << 20, dtype=torch.uint8, device=dev)      # larger than L2: written between steps
    chars = [0]
    found = [0]

    def steps(n, from_host):
        for i in range(n):
            host, devp, boxes = sets[i % 3]
            flush.fill_(i & 1)
            res = ocr.predict_pages(host if from_host else devp, boxes)
            chars[0] += sum(len(t) for r in res for t in r.text)
            found[0] += sum(len(b) for b in ocr.last_detected)
    sampler.wait_ready()
    warm = max(args.warmup, 3)
    steps(warm, False)
    steps(warm, True)
    ctx.barrier()
    sampler.rows.clear()
    l0 = ocr.gpu_launches
    dev_ms = ctx.time_blocks(lambda n: steps(n, False), args.steps, args.repeats)
    launches = (ocr.gpu_launches - l0) // (args.repeats * args.steps)
    e2e_ms = ctx.time_blocks(lambda n: steps(n, True), args.steps, args.repeats)
    h2d, d2h = ocr.h2d_bytes_last, ocr.d2h_bytes_last

    def flush_steps(n):
        for i in range(n):
            flush.fill_(i & 1)
    flush_ms = median(ctx.time_blocks(flush_steps, args.steps, 3))
    clocks = sampler.stop()
    ms_dev, ms_e2e = median(dev_ms) - flush_ms, median(e2e_ms) - flush_ms
    pages_total = B * ctx.world * args.steps
    non_native = sorted({s.name for st in (ocr.det, ocr.cls, ocr.rec) for p in st.rt._plans.values() for s in p.steps
                         if s.native is None})
    return {
        "metric": "pages/sec PP-OCRv3 det+cls+rec (device-timed)", "value": round(pages_total / (ms_dev / 1e3), 1),
        "unit": "pages/s", "n_gpus": ctx.world, "steps": args.steps, "warmup": warm,
        "ms_per_step": round(ms_dev / args.steps, 3), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "fp16", "data": "synthetic",
        "config": {"model": "PP-OCRv3 det (MobileNetV3 + RSE-FPN + DB head) + cls + rec (SVTR-LCNet, 6625 classes), "
                            "random-init weights",
                   "global_batch": B * ctx.world, "seq_len": None, "parallelism": f"dp{ctx.world}",
                   "page": f"{HW}x{HW} uint8, 20-60 boxes per page ({n_boxes / B:.1f} on average)",
                   "boxes": "classifier and recogniser read the synthetic layout's boxes (a random-init detector finds "
                            "no text); detector + device DB post-processing run on every page inside the timed region",
                   "buckets": "crop batches 8/16/32/64, recogniser widths 160/240/320/480/640/960",
                   "l2_policy": "192 MB written between steps (its own time, measured alone, is subtracted)",
                   "timing": f"median of {args.repeats} blocks of {args.steps} steps, CUDA events, max over ranks",
                   "baseline_ref": "the reference publishes no PP-OCR throughput"},
        "block_ms": spread(dev_ms),
        "e2e": {"value": round(pages_total / (ms_e2e / 1e3), 1), "unit": "pages/s", "h2d_bytes_per_step": int(h2d),
                "d2h_bytes_per_step": int(d2h), "ms_per_step": round(ms_e2e / args.steps, 3), "block_ms": spread(e2e_ms),
                "what": "DeviceOCR.predict_pages on a pinned page batch: pages and crop matrices in, box corners, "
                        "character ids and scores out"},
        "gpu_launches": int(launches), "non_native_steps": non_native,
        "boxes_per_step": round(n_boxes, 1), "detector_boxes_per_step": round(found[0] / max(1, (2 * warm + args.steps * args.repeats * 2)), 1),
        "clocks": clocks, "cpu_affinity": ctx.affinity, "impl": "ours",
    }
