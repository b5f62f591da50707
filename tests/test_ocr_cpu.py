"""PP-OCR pre/post-processing semantics and the three-stage pipeline on the CPU path."""
import numpy as np
import pytest


def test_ctc_greedy_decode():
    from fastdeploy_b200.vision.ocr import ctc_greedy_decode
    labels = ["#", "a", "b", "c", " "]
    idx = [1, 1, 0, 1, 2, 2, 3, 0, 0, 4]
    p = np.full((1, len(idx), 5), 0.01, np.float32)
    for t, k in enumerate(idx):
        p[0, t, k] = 0.9 - 0.01 * t
    text, score = ctc_greedy_decode(p, labels)
    assert text == ["aabc "]
    emitted = [0, 3, 4, 6, 9]
    assert score[0] == pytest.approx(np.mean([0.9 - 0.01 * t for t in emitted]), abs=1e-6)


def test_det_target_size_and_sort_boxes():
    from fastdeploy_b200.vision.ocr import DBDetectorPreprocessor, sort_boxes
    pre = DBDetectorPreprocessor()
    assert pre.target_hw(1080, 1920) == (544, 960)
    assert pre.target_hw(20, 20) == (32, 32)
    assert pre.target_hw(100, 333) == (96, 320)
    boxes = [[50, 12, 0, 0, 0, 0, 0, 0], [10, 15, 0, 0, 0, 0, 0, 0], [5, 60, 0, 0, 0, 0, 0, 0]]
    assert [b[0] for b in sort_boxes(boxes)] == [10, 50, 5]


def test_db_postprocess_finds_rectangles():
    from fastdeploy_b200.vision.ocr import DBDetectorPostprocessor
    prob = np.zeros((1, 1, 128, 256), np.float32)
    prob[0, 0, 20:40, 30:130] = 0.95
    prob[0, 0, 70:100, 150:240] = 0.9
    prob[0, 0, 110:112, 10:12] = 0.99           # too small
    post = DBDetectorPostprocessor()
    boxes = post.run(prob, [[512, 256, 256, 128]])[0]
    assert len(boxes) == 2
    b = sorted(boxes, key=lambda q: q[1])[0]
    xs, ys = b[0::2], b[1::2]
    # source image is 2x the map; the unclipped box must contain the blob and not be much larger
    assert min(xs) <= 60 and max(xs) >= 258 and min(ys) <= 40 and max(ys) >= 78
    assert max(xs) - min(xs) < 260 and max(ys) - min(ys) < 90


def test_rotate_crop():
    from fastdeploy_b200.vision.ocr import get_rotate_crop_image
    im = np.zeros((100, 200, 3), np.uint8)
    im[30:50, 40:140] = 200
    crop = get_rotate_crop_image(im, [40, 30, 139, 30, 139, 49, 40, 49])
    assert crop.shape[0] in (19, 20) and crop.shape[1] in (99, 100) and crop.mean() > 190
    tall = get_rotate_crop_image(im, [40, 10, 59, 10, 59, 89, 40, 89])
    assert tall.shape[1] > tall.shape[0]        # rotated to landscape


def test_ppocr_pipeline_cpu(tmp_path):
    import fastdeploy_b200 as fd
    from fastdeploy_b200.models.ppocr import write_ppocr
    paths = write_ppocr(str(tmp_path), vocab=64)
    opt = fd.RuntimeOption()
    opt.use_cpu()
    det = fd.vision.ocr.DBDetector(paths["det_model"], paths["det_params"], runtime_option=opt)
    cls = fd.vision.ocr.Classifier(paths["cls_model"], paths["cls_params"], runtime_option=opt)
    rec = fd.vision.ocr.Recognizer(paths["rec_model"], paths["rec_params"], paths["dict"], runtime_option=opt)
    assert len(rec.postprocessor.label_list) == 64
    det.postprocessor.det_db_thresh = 0.0         # random weights: make every pixel text so boxes exist
    det.postprocessor.det_db_box_thresh = 0.0
    ocr = fd.vision.ocr.PPOCRv3(det, cls, rec)
    im = np.random.RandomState(0).randint(0, 256, (96, 160, 3), dtype=np.uint8)
    res = ocr.predict(im)
    assert len(res.boxes) >= 1
    assert len(res.text) == len(res.boxes) == len(res.rec_scores) == len(res.cls_labels)
    assert "det boxes" in str(res)


def test_table_structure_decode_and_html(tmp_path):
    import numpy as np
    from fastdeploy_b200.vision.ocr import StructureV2TablePostprocessor, build_html
    p = tmp_path / "dict.txt"
    p.write_text("\n".join(["<thead>", "<tr>", "<td>", "</td>", "</tr>", "</thead>", "<td></td>", "beg", "end"]) + "\n")
    pp = StructureV2TablePostprocessor(str(p))
    assert pp.dict_character[0] == "sos" and pp.dict_character[-1] == "eos" and "<td>" not in pp.dict_character
    V, T = len(pp.dict_character), 8
    probs = np.zeros((1, T, V), np.float32)
    for i, t in enumerate(["beg", "<tr>", "<td></td>", "<td></td>", "</tr>", "eos", "<tr>"]):
        probs[0, i, pp.dict_character.index(t)] = 1
    boxes = np.zeros((1, T, 4), np.float32)
    boxes[0, 2] = [0.1, 0.1, 0.4, 0.3]
    boxes[0, 3] = [0.5, 0.1, 0.9, 0.3]
    b, t = pp.run(boxes, probs, [(1000, 500, 488, 244)])
    assert t[0] == ["<html>", "<body>", "<table>", "<tr>", "<td></td>", "<td></td>", "</tr>", "</table>", "</body>", "</html>"]
    assert b[0][0] == [100, 50, 400, 50, 400, 150, 100, 150]
    html = build_html(t[0], b[0], [[520, 60, 800, 60, 800, 140, 520, 140], [120, 55, 300, 55, 300, 145, 120, 145]], ["B", "A"])
    assert html == "<html><body><table><tr><td>A</td><td>B</td></tr></table></body></html>"


def test_layout_gfl_decode():
    import numpy as np
    from fastdeploy_b200.vision.ocr import StructureV2LayoutPostprocessor
    pp = StructureV2LayoutPostprocessor()
    in_w, in_h = 64, 64
    outs = []
    for s in pp.fpn_stride:
        a = int(np.ceil(in_w / s)) * int(np.ceil(in_h / s))
        outs.append(np.zeros((1, a, pp.num_class), np.float32))
    for s in pp.fpn_stride:
        a = int(np.ceil(in_w / s)) * int(np.ceil(in_h / s))
        outs.append(np.zeros((1, a, 4 * pp.reg_max), np.float32))
    outs[0][0, 8 * 3 + 4, 2] = 0.9                       # stride 8, cell (y=3, x=4)
    reg = np.full((4, pp.reg_max), -20.0, np.float32)
    reg[:, 2] = 20.0                                     # every distance = 2 strides
    outs[4][0, 8 * 3 + 4] = reg.reshape(-1)
    r = pp.run(outs, (128, 128, in_w, in_h))
    assert r.label_ids == [2] and abs(r.scores[0] - 0.9) < 1e-6
    assert np.allclose(r.boxes[0], [(36 - 16) * 2, (28 - 16) * 2, (36 + 16) * 2, (28 + 16) * 2], atol=1e-3)
