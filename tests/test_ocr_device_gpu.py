"""Device OCR stages against the host (OpenCV) path: DB post-processing, fused crop + resize + normalise, and the
GPU-resident pipeline."""
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rot_rect(cx, cy, w, h, deg):
    a = math.radians(deg)
    c, s = math.cos(a), math.sin(a)
    return np.array([[cx + dx * c - dy * s, cy + dx * s + dy * c]
                     for dx, dy in ((-w / 2, -h / 2), (w / 2, -h / 2), (w / 2, h / 2), (-w / 2, h / 2))], np.float32)


def _prob_map(h, w, rects, rng):
    import cv2
    prob = rng.uniform(0.0, 0.1, (h, w)).astype(np.float32)
    for (cx, cy, rw, rh, deg, level) in rects:
        mask = np.zeros((h, w), np.uint8)
        cv2.fillPoly(mask, [np.round(_rot_rect(cx, cy, rw, rh, deg)).astype(np.int32)], 1)
        prob[mask > 0] = level + rng.uniform(-0.02, 0.02, int(mask.sum())).astype(np.float32)
    return prob


@pytest.mark.parametrize("score_mode", ["slow", "fast"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_db_postprocess_matches_opencv_path(score_mode, dtype):
    from fastdeploy_b200.ops.postproc import DBPostprocess
    from fastdeploy_b200.vision.ocr import DBDetectorPostprocessor, sort_boxes
    rng = np.random.default_rng(0)
    H, W = 320, 480
    rect_sets = [
        [(100, 60, 150, 30, 0, 0.9), (300, 80, 120, 24, 12, 0.85), (240, 200, 200, 36, -20, 0.95), (60, 260, 80, 20, 45, 0.9),
         (400, 270, 40, 90, 3, 0.8), (20, 20, 2, 2, 0, 0.9), (430, 40, 60, 20, 0, 0.5)],     # tiny: dropped; 0.5: below box_thresh
        [(240, 160, 300, 60, 7, 0.92), (90, 40, 100, 18, -4, 0.7), (380, 280, 120, 40, 30, 0.88)],
    ]
    maps = np.stack([_prob_map(H, W, r, rng) for r in rect_sets])
    infos = [(960, 640, W, H), (480, 300, W - 32, H - 16)]          # source sizes and valid map regions
    host = DBDetectorPostprocessor()
    host.det_db_score_mode = score_mode
    want = [sort_boxes(b) for b in host.run(maps[:, None], infos)]
    # an NHWC single-channel map padded to 8 channels, as the detector's plan produces it
    buf = torch.zeros(2, H, W, 8, dtype=dtype, device="cuda")
    buf[..., 0] = torch.from_numpy(maps).cuda().to(dtype)
    db = DBPostprocess(2, H, W, "cuda", score_mode=score_mode)
    db.set_info(infos)
    for _ in range(2):                                  # a second run reuses the scratch
        db.run(buf[..., 0])
    got, scores = db.boxes()
    got = [sort_boxes(b) for b in got]
    assert [len(b) for b in got] == [len(b) for b in want] == [5, 3]
    for g, w_ in zip(got, want):
        diff = np.abs(np.asarray(g) - np.asarray(w_))
        assert diff.max() <= 2, (g, w_)
        assert (diff <= 1).mean() > 0.9
    assert all(0.6 <= s <= 1.0 for sl in scores for s in sl)


def test_db_postprocess_handles_noise_and_empty_maps():
    from fastdeploy_b200.ops.postproc import DBPostprocess
    rng = np.random.default_rng(1)
    H, W = 160, 160
    maps = torch.from_numpy(np.stack([rng.uniform(0, 1, (H, W)), np.zeros((H, W))]).astype(np.float32)).cuda()
    db = DBPostprocess(2, H, W, "cuda", max_candidates=100)      # far more than 100 specks in the noise map
    db.set_info([(W, H, W, H)] * 2)
    db.run(maps)
    torch.cuda.synchronize()
    boxes, _ = db.boxes()
    assert boxes[1] == [] and len(boxes[0]) <= 100
    for b in boxes[0]:
        assert all(0 <= v < W for v in b)


def test_warp_normalize_matches_crop_resize_normalize():
    import cv2
    from fastdeploy_b200.ops import postproc as PP
    from fastdeploy_b200.vision.ocr import get_rotate_crop_image
    rng = np.random.default_rng(2)
    H, W = 300, 500
    yy, xx = np.mgrid[0:H, 0:W]
    page = np.stack([(xx * 0.4 + yy * 0.2) % 256, (xx * 0.1 + 60 + 40 * np.sin(yy / 23.0)) % 256, (yy * 0.7) % 256], -1)
    page = cv2.GaussianBlur(page.astype(np.uint8), (0, 0), 2.0)
    pages = np.stack([page, page[::-1].copy()])
    boxes = [[40, 50, 260, 60, 258, 100, 38, 90], [300, 40, 330, 40, 330, 200, 300, 200], [100, 150, 400, 150, 400, 190, 100, 190]]
    page_idx = np.array([0, 1, 1], np.int32)
    mats, vw, ratios = PP.crop_matrices(boxes, 48, 320)
    out = torch.zeros(4, 48, 320, 8, dtype=torch.float16, device="cuda")
    vw_full = np.zeros(4, np.int32)
    vw_full[:3] = vw
    flip = torch.tensor([0, 0, 1, 0], dtype=torch.int32, device="cuda")
    mat_full = np.zeros((4, 9), np.float32)
    mat_full[:3] = mats
    PP.warp_normalize_batch(torch.from_numpy(pages).cuda(), torch.from_numpy(mat_full).cuda(), torch.from_numpy(vw_full).cuda(),
                            out, [2 / 255.0] * 3, [-1.0] * 3, flip=flip,
                            page=torch.from_numpy(np.concatenate([page_idx, [0]]).astype(np.int32)).cuda())
    torch.cuda.synchronize()
    got = out.float().cpu().numpy()
    assert np.abs(got[3]).max() == 0 and np.abs(got[..., 3:]).max() == 0
    for i, box in enumerate(boxes):
        crop = get_rotate_crop_image(pages[page_idx[i]], box)
        rw = int(vw[i])
        ref = cv2.resize(crop, (rw, 48)).astype(np.float32) / 255.0 * 2 - 1
        if i == 2:
            ref = ref[::-1, ::-1]
        assert abs(crop.shape[1] / crop.shape[0] - ratios[i]) < 0.05
        assert rw == 320 or np.abs(got[i, :, rw:]).max() == 0
        err = np.abs(got[i, :, :rw, :3] - ref)
        assert err.mean() < 0.03 and np.percentile(err, 99) < 0.15, (i, err.mean(), err.max())


def test_device_pipeline_runs_all_stages_on_the_gpu(tmp_path):
    import fastdeploy_b200 as fd
    from fastdeploy_b200.benchmarks.ocr import make_pages
    from fastdeploy_b200.models import ppocr
    from fastdeploy_b200.vision.ocr.device_pipeline import DeviceOCR
    paths = ppocr.write_ppocr(str(tmp_path), vocab=97)

    def option():
        o = fd.RuntimeOption()
        o.use_gpu(0)
        o.enable_trt_fp16()
        return o
    det = fd.vision.ocr.DBDetector(paths["det_model"], paths["det_params"], runtime_option=option())
    cls = fd.vision.ocr.Classifier(paths["cls_model"], paths["cls_params"], runtime_option=option())
    rec = fd.vision.ocr.Recognizer(paths["rec_model"], paths["rec_params"], paths["dict"], runtime_option=option())
    pages, boxes = make_pages(np.random.default_rng(3), 2, 320)
    boxes = [b[:13] for b in boxes]
    ocr = DeviceOCR(det, cls, rec, rec_widths=(160, 320, 640), batches=(8, 16))
    res = ocr.predict_pages(pages, boxes)
    assert [len(r.text) for r in res] == [13, 13] and [len(r.cls_labels) for r in res] == [13, 13]
    assert all(isinstance(t, str) for r in res for t in r.text)
    assert all(0.0 <= s <= 1.0 for r in res for s in r.rec_scores)
    for st in (ocr.det, ocr.cls, ocr.rec):
        for plan in st.rt._plans.values():
            assert [s.name for s in plan.steps if s.native is None] == []
    # the same pages again from a device tensor give the same text
    res2 = ocr.predict_pages(torch.from_numpy(pages).cuda(), boxes)
    assert [r.text for r in res2] == [r.text for r in res]
    # the recogniser's answer for one crop equals a direct run of its plan on the same crop pixels
    pipe = fd.vision.ocr.PPOCRv3(det, cls, rec)
    out = pipe.batch_predict([pages[0], pages[1]])       # detector boxes (whatever a random net finds): must not fail
    assert len(out) == 2 and all(len(r.text) == len(r.boxes) for r in out)
