"""Decoders of the model families on hand-made network outputs (no runtime involved)."""
import numpy as np
import pytest

from fastdeploy_b200.vision.detection import contrib as C
from fastdeploy_b200.vision import facedet, keypointdetection as K, perception as P, tracking as T, utils as U


def test_letterbox_geometry_and_inverse():
    img = np.zeros((480, 640, 3), np.uint8)
    canvas, info = C.letterbox(img, (640, 640))
    assert canvas.shape == (640, 640, 3) and info["pad_h"] == 80 and info["pad_w"] == 0 and info["scale"] == 1.0
    assert (canvas[:80] == 114).all() and (canvas[80:560] == 0).all()
    canvas, info = C.letterbox(np.zeros((100, 50, 3), np.uint8), (64, 64), scale_up=False)
    assert info["scale"] == 0.64 and canvas.shape == (64, 64, 3)


def test_yolov5_decode_class_aware_nms():
    _, infos = C.YOLOPreprocessor().run([np.zeros((480, 640, 3), np.uint8)])
    out = np.zeros((1, 10, 85), np.float32)
    out[0, 0, :5] = [320, 320, 100, 80, 0.9]; out[0, 0, 5 + 3] = 0.8
    out[0, 1, :5] = [322, 321, 100, 80, 0.8]; out[0, 1, 5 + 3] = 0.9     # same class, suppressed
    out[0, 2, :5] = [322, 321, 100, 80, 0.8]; out[0, 2, 5 + 7] = 0.9     # other class, kept
    r = C.YOLOPostprocessor("v5").run([out], infos)[0]
    assert sorted(r.label_ids) == [3, 7] and len(r.boxes) == 2
    b = r.boxes[r.label_ids.index(3)]
    assert np.allclose(b, [270, 200, 370, 280])          # letterbox padding of 80 rows removed


def test_yolov8_and_yolox_layouts():
    _, infos = C.YOLOPreprocessor().run([np.zeros((640, 640, 3), np.uint8)])
    out8 = np.zeros((1, 84, 5), np.float32)
    out8[0, :4, 0] = [100, 100, 40, 40]; out8[0, 4 + 2, 0] = 0.7
    r = C.YOLOPostprocessor("v8").run([out8], infos)[0]
    assert r.label_ids == [2] and np.allclose(r.boxes[0], [80, 80, 120, 120])
    pp = C.YOLOPostprocessor("x")
    n = sum((640 // s) ** 2 for s in pp.strides)
    outx = np.zeros((1, n, 85), np.float32)
    outx[0, 81, :5] = [0.5, 0.5, np.log(4.0), np.log(2.0), 0.9]; outx[0, 81, 5] = 0.9    # cell (1, 1) of stride 8
    r = pp.run([outx], infos)[0]
    assert np.allclose(r.boxes[0], [(1.5 * 8) - 16, (1.5 * 8) - 8, (1.5 * 8) + 16, (1.5 * 8) + 8].copy() if False else
                       [max(0, 12 - 16), 12 - 8, 12 + 16, 12 + 8])


def test_scrfd_decode_with_landmarks():
    m = facedet.SCRFD.__new__(facedet.SCRFD)
    m.size = [64, 64]; m.conf_threshold = 0.5; m.nms_iou_threshold = 0.4
    facedet.SCRFD._configure(m)
    info = {"scale": 1.0, "pad_w": 0, "pad_h": 0, "in_hw": (64, 64), "out_hw": (64, 64)}
    outs = []
    for s in m.strides:
        n = (64 // s) ** 2 * 2
        outs.append(np.zeros((n, 1), np.float32))
    for s in m.strides:
        outs.append(np.zeros(((64 // s) ** 2 * 2, 4), np.float32))
    for s in m.strides:
        outs.append(np.zeros(((64 // s) ** 2 * 2, 10), np.float32))
    outs[0][2 * (8 * 2 + 3), 0] = 0.9                      # stride 8, cell (y=2, x=3), anchor 0
    outs[3][2 * (8 * 2 + 3)] = [1, 1, 2, 2]
    outs[6][2 * (8 * 2 + 3)] = [0.5] * 10
    r = m.postprocess(outs, info)
    assert len(r.boxes) == 1 and np.allclose(r.boxes[0], [24 - 8, 16 - 8, 24 + 16, 16 + 16])
    assert r.landmarks_per_face == 5 and np.allclose(r.landmarks[0], [28, 20])


def test_dark_and_plain_heatmap_decoding_agree_on_symmetric_peak():
    heat = np.zeros((1, 32, 24), np.float32)
    yy, xx = np.mgrid[0:32, 0:24]
    heat[0] = np.exp(-((xx - 10) ** 2 + (yy - 12) ** 2) / 4.0)
    p1, s1 = K.decode_heatmaps(heat, (50, 60), (48, 64), use_dark=True)
    p2, s2 = K.decode_heatmaps(heat, (50, 60), (48, 64), use_dark=False)
    assert np.allclose(p1, p2, atol=0.6) and abs(s1[0] - 1) < 1e-6
    m, mi = K.get_affine((100, 80), (60, 80), (192, 256)), K.get_affine((100, 80), (60, 80), (192, 256), inv=True)
    assert np.allclose(mi @ np.r_[m @ [100, 80, 1], 1], [100, 80], atol=1e-3)


def test_trackers_keep_identities():
    rng = np.random.default_rng(0)
    f = rng.standard_normal((2, 16))
    jt, oc = T.JDETracker(), T.OCSortTracker(det_thresh=0.3)
    ids_j, ids_o = [], []
    for fr in range(10):
        b = np.array([[100 + 5 * fr, 100, 150 + 5 * fr, 200], [300, 50 + 3 * fr, 380, 190 + 3 * fr]], float)
        if fr == 4:            # one missed detection in the middle
            b = b[:1]
            tr = jt.update(b, np.array([0.9]), f[:1])
            o = oc.update(b, np.array([0.9]))
        else:
            tr = jt.update(b, np.array([0.9, 0.8]), f + 0.01 * rng.standard_normal((2, 16)))
            o = oc.update(b, np.array([0.9, 0.8]))
        ids_j.append(sorted(t.id for t in tr)); ids_o.append(sorted(int(i) for i in o[:, 4]))
    assert ids_j[-1] == ids_j[0] and len(ids_j[0]) == 2
    assert ids_o[-1] == ids_o[0] and len(ids_o[0]) == 2


def test_voxelize_and_bev_nms():
    pts = np.array([[0.1, 0.1, 0, 1], [0.2, 0.2, 0, 1], [0.3, 0.3, 0, 1], [5.1, 5.1, 0, 1], [99, 0, 0, 1]], np.float32)
    v, c, n = P.hard_voxelize(pts, [1, 1, 8], [0, 0, -4, 10, 10, 4], max_points=2, max_voxels=10)
    assert v.shape == (2, 2, 4) and n.tolist() == [2, 1] and c.tolist() == [[0, 0, 0], [0, 5, 5]]
    assert abs(P.rotated_iou_bev((0, 0, 2, 4, 0), (1, 0, 2, 4, 0)) - 1 / 3) < 1e-6
    assert abs(P.rotated_iou_bev((0, 0, 2, 2, 0), (0, 0, 2, 2, np.pi / 4)) - 0.70710678) < 1e-4
    boxes = np.array([[0, 0, 2, 4, 0], [0.2, 0, 2, 4, 0], [10, 10, 2, 4, 1.0]], np.float32)
    assert P.nms_bev(boxes, np.array([0.9, 0.8, 0.7]), 0.5) == [0, 2]


def test_detection_postprocessor_rotated_masks_and_solov2():
    from fastdeploy_b200.ops.perception import multiclass_nms_rotated_numpy
    from fastdeploy_b200.vision.detection.ppdet import NMSOption, PaddleDetPostprocessor
    rng = np.random.default_rng(0)
    # PP-YOLOE-R: [N, M, 8] quadrilaterals + [N, C, M] scores -> rotated boxes divided by the resize factors
    quads = np.array([[10, 10, 50, 10, 50, 30, 10, 30], [12, 11, 52, 11, 52, 31, 12, 31], [100, 100, 140, 120, 130, 140, 90, 120]],
                     np.float32)
    scores = np.array([[0.9, 0.8, 0.1], [0.05, 0.02, 0.7]], np.float32)
    post = PaddleDetPostprocessor()
    opt = NMSOption()
    opt.score_threshold, opt.nms_threshold, opt.nms_top_k, opt.keep_top_k = 0.3, 0.3, 100, 10
    post.set_nms_rotated_option(opt)
    post.set_scale_factor([2.0, 4.0])
    res = post.run([quads[None], scores[None]])[0]
    assert res.label_ids == [0, 1] and [round(s, 2) for s in res.scores] == [0.9, 0.7]     # box 1 is suppressed by box 0
    assert res.rotated_boxes[0] == [2.5, 5.0, 12.5, 5.0, 12.5, 15.0, 2.5, 15.0]
    rows, idx = multiclass_nms_rotated_numpy(quads, scores, 0.3, 0.3, 100, 10)
    assert idx.tolist() == [0, 2] and rows.shape == (2, 10)
    # Mask R-CNN: the third output is one full-image mask per box, cropped to the rounded box
    boxes = np.array([[1, 0.9, 2.2, 3.4, 6.1, 7.0], [0, 0.8, 0.0, 0.0, 4.0, 2.0]], np.float32)
    masks = rng.integers(0, 2, (2, 10, 12)).astype(np.int32)
    post = PaddleDetPostprocessor()
    res = post.run([boxes, np.array([2], np.int32), masks])[0]
    assert res.contain_masks and res.masks[0].shape == [4, 4] and res.masks[1].shape == [2, 4]
    assert res.masks[0].data == masks[0, 3:7, 2:6].reshape(-1).tolist()
    assert res.masks[1].data == masks[1, 0:2, 0:4].reshape(-1).tolist()
    # SOLOv2: count, labels, scores, masks -> boxes are the mask extents
    m = np.zeros((3, 8, 9), np.uint8)
    m[0, 2:5, 1:7] = 1
    m[1, 0:2, 3:4] = 1
    m[2, 6:8, 6:9] = 1
    post = PaddleDetPostprocessor("SOLOv2")
    post.nms_option.score_threshold = 0.5
    res = post.run([np.array([3], np.int32), np.array([4, 5, 6], np.int64), np.array([0.9, 0.2, 0.6], np.float32), m])[0]
    assert res.label_ids == [4, 6] and res.boxes == [[1.0, 2.0, 7.0, 5.0], [6.0, 6.0, 9.0, 8.0]]
    assert res.masks[0].shape == [3, 6] and sum(res.masks[0].data) == 18 and res.masks[1].shape == [2, 3]


def test_ser_vi_layoutxlm_windows_reading_order_and_line_vote(tmp_path):
    from fastdeploy_b200.vision.ocr import ser as S

    class Tok:                       # one id per character, wrapped in cls / sep like a real tokenizer
        def encode(self, text):
            return [0] + [10 + ord(c) % 50 for c in text] + [2]

    (tmp_path / "cls.txt").write_text("OTHER\nQUESTION\nANSWER\nHEADER\n")
    labels = S.load_labels(str(tmp_path / "cls.txt"))
    assert labels == ["O", "B-QUESTION", "I-QUESTION", "B-ANSWER", "I-ANSWER", "B-HEADER", "I-HEADER"]
    lines = [{"bbox": [300, 105, 400, 130], "transcription": "bb"},
             {"bbox": [10, 100, 200, 130], "transcription": "aaa"},          # same row, further left: comes first
             {"bbox": [10, 10, 20, 30, 20, 40, 10, 40], "transcription": "h"},
             {"bbox": [10, 400, 600, 430], "transcription": "c" * 600}]      # spills into a second window
    pre = S.StructureV2SERViLayoutXLMPreprocessor(Tok(), max_seq_len=512)
    b = pre.run(lines, height=500, width=1000)
    assert [r["transcription"][:1] for r in b["ocr_info"]] == ["h", "a", "b", "c"]
    assert b["segment_offset_id"] == [1, 4, 6, 606]
    assert b["input_ids"].shape == (2, 512) and b["bbox"].shape == (2, 512, 4)
    assert b["input_ids"][0, 0] == 0 and b["input_ids"][0, 511] == 2 and b["attention_mask"][0].sum() == 512
    assert b["attention_mask"][1].sum() == 606 - 510 + 2 and b["input_ids"][1, 97] == 2 and b["input_ids"][1, 98] == 1
    assert b["bbox"][0, 1].tolist() == [10, 20, 20, 80]                       # 8-number box -> xyxy on the 0..1000 grid
    assert b["bbox"][0, 2].tolist() == [10, 200, 200, 260] and b["bbox"][1, 97].tolist() == [1000] * 4

    post = S.StructureV2SERViLayoutXLMPostprocessor(labels=labels)
    assert post.draw_names == ["O", "QUESTION", "ANSWER", "HEADER"]
    logits = np.zeros((2, 512, len(labels)), np.float32)
    logits[..., 0] = 0.1
    logits[0, 1, 5] = 1                                   # "h": B-HEADER
    logits[0, 2, 1] = 1; logits[0, 3, 2] = 1              # "aaa": B-Q, I-Q, O -> QUESTION
    logits[0, 5, 3] = 1; logits[0, 6, 4] = 1              # "bb": B-A, I-A
    logits[1, 1:97, 4] = 1                                # tail of the long line: 96 x I-ANSWER against 504 x O
    r = post.run(logits, b)
    assert r.pred == ["HEADER", "QUESTION", "ANSWER", "O"] and r.pred_id == [3, 1, 2, 0]

    m = S.StructureV2SERViLayoutXLM.__new__(S.StructureV2SERViLayoutXLM)
    m.preprocessor, m.postprocessor, m.ocr = pre, post, None

    class Info:
        def __init__(self, n): self.name = n

    class FakeRuntime:
        def num_inputs(self): return 4
        def get_input_info(self, i): return Info(["x0", "x1", "x2", "x3"][i])
        def infer(self, feeds):
            assert feeds["x1"].shape == (4, 512, 4) and feeds["x0"].dtype == np.int64
            return [np.concatenate([logits, logits])]
    m.runtime = FakeRuntime()
    two = m.batch_predict([np.zeros((500, 1000, 3), np.uint8)] * 2, [lines, lines])
    assert [x.pred for x in two] == [r.pred, r.pred]
    with pytest.raises(ValueError):
        m.predict(np.zeros((500, 1000, 3), np.uint8))


def test_ser_vi_layoutxlm_runs_a_model_end_to_end(tmp_path):
    """The SER class on a synthetic vi-LayoutXLM export (CPU runtime): windows in, one label per text line out, the
    same labels as arg-max + line vote done by hand on the runtime's logits."""
    import fastdeploy_b200 as fd
    from fastdeploy_b200.models.layoutxlm import write_ser_vi_layoutxlm
    from fastdeploy_b200.vision.ocr import StructureV2SERViLayoutXLM
    paths = write_ser_vi_layoutxlm(str(tmp_path), "tiny", num_labels=7, seed=3)

    class Tok:
        def encode(self, text):
            return [0] + [3 + ord(c) % 250 for c in text] + [2]
    opt = fd.RuntimeOption()
    opt.use_cpu()
    m = StructureV2SERViLayoutXLM(paths["model"], paths["params"], paths["classes"], tokenizer=Tok(), runtime_option=opt)
    assert m.initialized and m.postprocessor.draw_names == ["O", "QUESTION", "ANSWER", "HEADER"]
    lines = [{"bbox": [40, 30, 400, 60], "transcription": "Invoice number"},
             {"bbox": [420, 30, 700, 60], "transcription": "2024-117"},
             {"bbox": [40, 90, 300, 120], "transcription": "Total amount due"},
             {"bbox": [40, 200, 900, 230], "transcription": "x" * 700}]            # forces a second window
    page = np.zeros((400, 1000, 3), np.uint8)
    res = m.predict(page, lines)
    assert len(res.pred) == 4 and all(p in m.postprocessor.draw_names for p in res.pred)
    assert res.text[0] == "Invoice number" and res.boxes[1] == [420, 30, 700, 60]
    batch = m.preprocessor.run(lines, 400, 1000)
    assert batch["input_ids"].shape == (2, 512)
    feeds = {"input_ids": batch["input_ids"], "bbox": batch["bbox"], "attention_mask": batch["attention_mask"],
             "token_type_ids": batch["token_type_ids"]}
    logits = m.runtime.infer(feeds)[0]
    assert logits.shape == (2, 512, 7)
    by_hand = m.postprocessor.run(logits, batch)
    assert by_hand.pred == res.pred and by_hand.pred_id == res.pred_id
    two = m.batch_predict([page, page], [lines, lines[:2]])
    assert two[0].pred == res.pred and two[1].pred == res.pred[:2] or len(two[1].pred) == 2


def test_native_hard_nms_matches_the_numpy_scan():
    rng = np.random.default_rng(5)
    for n, thr in ((1, 0.5), (50, 0.3), (800, 0.6)):
        c = rng.random((n, 2)) * 100
        wh = rng.random((n, 2)) * 30 + 2
        boxes = np.concatenate([c - wh / 2, c + wh / 2], 1).astype(np.float32)
        scores = np.round(rng.random(n), 1).astype(np.float32)                 # many ties: the order must be stable
        got = U.nms_indices(boxes, scores, thr)
        want = U._nms_indices_numpy(boxes, scores, thr)
        assert np.array_equal(got, want)
        assert np.array_equal(U.nms_indices(boxes, scores, thr, max_keep=3), want[:3])
    assert U.nms_indices(np.zeros((0, 4), np.float32), np.zeros(0, np.float32)).size == 0


def test_ser_model_under_the_reference_constructor_order(tmp_path):
    from fastdeploy_b200.core.types import ModelFormat
    from fastdeploy_b200.models.layoutxlm import write_ser_vi_layoutxlm
    from fastdeploy_b200.runtime.option import RuntimeOption
    from fastdeploy_b200.vision.ocr import StructureV2SERViLayoutXLM, StructureV2SERViLayoutXLMModel

    class Tok:
        def encode(self, text):
            return [5 + (ord(c) % 50) for c in text if not c.isspace()]

    paths = write_ser_vi_layoutxlm(str(tmp_path), "tiny", num_labels=7, seed=3)
    opt = RuntimeOption(); opt.use_cpu()
    a = StructureV2SERViLayoutXLM(paths["model"], paths["params"], paths["classes"], tokenizer=Tok(), runtime_option=opt)
    b = StructureV2SERViLayoutXLMModel(paths["model"], paths["params"], "rec_dict.txt", paths["classes"], "", opt, ModelFormat.PADDLE,
                                       tokenizer=Tok())
    assert b.ser_dict_path == "rec_dict.txt" and b.postprocesser is b.postprocessor
    im = np.zeros((200, 300, 3), np.uint8)
    lines = [{"bbox": [10, 10, 120, 30], "transcription": "name"}, {"points": [[10, 50], [150, 50], [150, 70], [10, 70]], "transcription": "alice"}]
    ra, rb = a.predict(im, lines), b.predict(im, lines)
    assert ra.pred == rb.pred and ra.text == rb.text == ["name", "alice"]
