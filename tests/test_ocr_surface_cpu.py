"""OCR classes' switches and helper operators that user code written for the reference relies on."""
import numpy as np
import pytest

import fastdeploy_b200 as fd

ocr = fd.vision.ocr


def _img(h, w, seed=0):
    return np.random.default_rng(seed).integers(0, 255, (h, w, 3), dtype=np.uint8)


def test_preprocessor_switches_on_the_three_stages():
    im = _img(40, 100)
    for make in (ocr.ClassifierPreprocessor, ocr.RecognizerPreprocessor):
        base = make().run([im])
        p = make(); p.disable_permute()
        assert np.allclose(p.run([im]).transpose(0, 3, 1, 2), base)
        p = make(); p.disable_normalize()
        raw = p.run([im])
        assert raw.max() > 2 and np.allclose((raw / 255.0 - 0.5) / 0.5, base, atol=1e-5) or make is ocr.ClassifierPreprocessor
        p = make(); p.set_normalize([0.0] * 3, [1.0] * 3, False)
        assert p.run([im]).max() > 2                     # neither scaled nor shifted
    d = ocr.DBDetectorPreprocessor()
    base, info = d.run([im])
    assert base.shape == (1, 3, 32, 96) and info == [[100, 40, 96, 32]]
    d2 = ocr.DBDetectorPreprocessor(); d2.disable_normalize(); d2.disable_permute()
    raw, _ = d2.run([im])
    assert raw.shape == (1, 32, 96, 3) and raw.max() > 2
    assert np.allclose(((raw / 255.0 - np.float32(d.mean)) / np.float32(d.scale)).transpose(0, 3, 1, 2), base, atol=1e-4)


def test_model_level_names_of_older_releases():
    det = ocr.DBDetector.__new__(ocr.DBDetector)
    det.preprocessor, det.postprocessor = ocr.DBDetectorPreprocessor(), ocr.DBDetectorPostprocessor()
    det.det_db_thresh, det.det_db_box_thresh, det.det_db_unclip_ratio = 0.2, 0.5, 2.0
    det.det_db_score_mode, det.use_dilation, det.max_side_len = "fast", True, 640
    pp = det.postprocessor
    assert (pp.det_db_thresh, pp.det_db_box_thresh, pp.det_db_unclip_ratio, pp.det_db_score_mode, pp.use_dilation) == \
        (0.2, 0.5, 2.0, "fast", True) and det.preprocessor.max_side_len == 640
    cls = ocr.Classifier.__new__(ocr.Classifier)
    cls.preprocessor, cls.postprocessor = ocr.ClassifierPreprocessor(), ocr.ClassifierPostprocessor()
    cls.cls_thresh, cls.cls_image_shape = 0.8, [3, 32, 128]
    assert cls.postprocessor.cls_thresh == 0.8 and cls.preprocessor.run([_img(20, 50)]).shape == (1, 3, 32, 128)
    rec = ocr.Recognizer.__new__(ocr.Recognizer)
    rec.preprocessor = ocr.RecognizerPreprocessor()
    rec.rec_image_shape, rec.static_shape_infer = [3, 32, 100], True
    assert rec.preprocessor.run([_img(20, 400)]).shape == (1, 3, 32, 100)
    assert ocr.PPStructureV2TableSystem is ocr.PPStructureV2Table
    assert issubclass(ocr.StructureV2SERViLayoutXLMModel, ocr.StructureV2SERViLayoutXLM)
    with pytest.raises(ValueError, match="sentencepiece.bpe.model"):
        ocr.StructureV2SERViLayoutXLMModel("/nonexistent/model.pdmodel", "", "dict.txt", "classes.txt")
    post = fd.vision.segmentation.PaddleSegPostprocessor
    assert post().is_with_argmax and not post(False, True).is_with_argmax and post(False, True).is_with_softmax


def test_layout_preprocessor_and_table_pipeline_batches():
    pre = ocr.StructureV2LayoutPreprocessor()
    x = pre.run([_img(100, 200), _img(50, 60, 1)])
    assert x.shape == (2, 3, 800, 608) and pre.batch_layout_img_info == [(200, 100, 608, 800), (60, 50, 608, 800)]

    class Stage:
        def __init__(self, tag): self.tag = tag
        def clone(self): return Stage(self.tag + "'")

    seen = []

    class Table(ocr.PPStructureV2Table):
        def predict(self, im):
            seen.append(im.shape)
            return im.shape[0]

    t = Table(Stage("det"), Stage("rec"), Stage("table"))
    assert t.batch_predict([_img(10, 20), _img(30, 20)]) == [10, 30] and len(seen) == 2
    c = ocr.PPStructureV2Table(Stage("det"), Stage("rec"), Stage("table")).clone()
    assert (c.detector.tag, c.recognizer.tag, c.table.tag) == ("det'", "rec'", "table'")


class _WordTokenizer:
    """One id per whitespace-separated word, stable across calls."""

    def __init__(self):
        self.vocab = {}

    def encode(self, text):
        return [self.vocab.setdefault(w, 10 + len(self.vocab)) for w in text.split()]


def test_token_pipeline_operators_agree_with_the_one_call_preprocessor():
    lines = [{"bbox": [10, 50, 110, 70], "transcription": "total amount due"},
             {"points": [[10, 10], [90, 10], [90, 30], [10, 30]], "transcription": "invoice number"},
             {"bbox": [150, 10, 300, 30], "transcription": "A 1234"},
             {"bbox": [0, 0, 5, 5], "transcription": ""}]
    page = {"image": _img(100, 400), "ocr_info": lines}
    tok = _WordTokenizer()
    data = ocr.VQATokenLabelEncode(tok)(dict(page))
    assert [r["transcription"] for r in data["ocr_info"]] == ["invoice number", "A 1234", "total amount due"]   # reading order
    assert data["segment_offset_id"] == [2, 4, 7] and len(data["input_ids"]) == 7
    assert data["bbox"][0] == [25, 100, 225, 300] and data["bbox"][2] == [375, 100, 750, 300]
    padded = ocr.VQATokenPad(max_seq_len=5, pad_to_max_seq_len=True)(dict(data))
    assert padded["input_ids"].dtype == np.int64 and padded["bbox"].shape == (7, 4)       # longer than the window: untouched
    chunks = ocr.VQASerTokenChunk(max_seq_len=5)(padded)
    assert chunks["input_ids"].shape == (2, 5) and chunks["bbox"].shape == (2, 5, 4)
    assert chunks["attention_mask"].tolist() == [[1] * 5, [1, 1, 0, 0, 0]]
    short = ocr.VQATokenPad(max_seq_len=16)(ocr.VQATokenLabelEncode(tok)(dict(page)))
    assert short["input_ids"].shape == (16,) and short["input_ids"][7:].tolist() == [1] * 9
    # the same page through the model's own pre-processor: identical tokens and boxes, framed by CLS / SEP
    ref = ocr.StructureV2SERViLayoutXLMPreprocessor(tok, max_seq_len=16).run(lines[:3], 100, 400)
    assert ref["input_ids"][0, 1:8].tolist() == short["input_ids"][:7].tolist()
    assert ref["bbox"][0, 1:8].tolist() == short["bbox"][:7].tolist() and ref["segment_offset_id"] == data["segment_offset_id"]
    # the vote: logits that say class 1 for the first line's tokens, class 2 for the rest
    labels = ["O", "B-QUESTION", "I-QUESTION", "B-ANSWER", "I-ANSWER"]
    logits = np.zeros((1, 16, 5), np.float32)
    logits[0, 0:2, 1] = 5; logits[0, 2:4, 3] = 5; logits[0, 4:7, 2] = 5
    post = ocr.VQASerTokenLayoutLMPostProcess(labels=labels)
    out = post(logits, segment_offset_ids=[data["segment_offset_id"]], ocr_infos=[data["ocr_info"]])[0]
    assert [r["pred"] for r in out] == ["QUESTION", "ANSWER", "QUESTION"] and out[1]["transcription"] == "A 1234"
    # image operators
    d = ocr.Resize(size=(50, 100))({"image": _img(100, 400)})
    assert d["image"].shape == (50, 100, 3)
    d = ocr.ToCHWImage()(ocr.NormalizeImage(scale="1./255.", mean=[0.5] * 3, std=[0.5] * 3, order="hwc")(d))
    assert d["image"].shape == (3, 50, 100) and -1.0 <= d["image"].min() and d["image"].max() <= 1.0
    assert ocr.KeepKeys(["image", "resized_shape"])(d)[1] == [50, 100]
    # relation extraction: entities past the window and their relations are dropped
    re = ocr.VQATokenLabelEncode(tok, contains_re=True)(dict(page, relations=[{"head": 0, "tail": 1}, {"head": 0, "tail": 2}]))
    cut = ocr.VQAReTokenChunk(max_seq_len=4)(re)
    assert cut["entities"]["end"] == [2, 4] and cut["relations"] == {"head": [0], "tail": [1]} and len(cut["input_ids"]) == 4
