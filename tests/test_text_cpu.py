"""Tokenizer (C++ vs Python mirror), UIE decoding rules and the ERNIE runners on CPU."""
import os

import numpy as np
import pytest

from fastdeploy_b200.text.tokenizer import ErnieTokenizer, PyErnieTokenizer, write_synthetic_vocab
from fastdeploy_b200.text import uie as U


@pytest.fixture(scope="module")
def vocab(tmp_path_factory):
    p = str(tmp_path_factory.mktemp("tok") / "vocab.txt")
    write_synthetic_vocab(p, 30000)
    return p


def test_wordpiece_rules(vocab):
    t = PyErnieTokenizer(vocab)
    e = t.encode("Hello, World", "时间2023")
    v = t.vocab
    assert e.ids[0] == v["[CLS]"] and e.ids.count(v["[SEP]"]) == 2
    assert e.type_ids[:e.ids.index(v["[SEP]"]) + 1] == [0] * (e.ids.index(v["[SEP]"]) + 1)
    assert e.type_ids[-1] == 1
    # offsets are per segment, specials carry (0, 0), a CJK character is one token
    sep = e.ids.index(v["[SEP]"])
    assert e.offsets[0] == (0, 0) and e.offsets[sep] == (0, 0)
    assert e.offsets[sep + 1] == (0, 1) and e.offsets[sep + 2] == (1, 2)
    assert e.ids[sep + 1] == v["时"]
    # lower-casing: "Hello" and "hello" agree
    assert t.encode("Hello").ids == t.encode("hello").ids
    # accent stripping for Latin-1
    assert t.encode("café").ids == t.encode("cafe").ids
    # a comma is its own token
    toks = t.encode("a,b")
    assert len(toks.ids) == 5


def test_truncation_longest_first(vocab):
    t = PyErnieTokenizer(vocab)
    e = t.encode("一二三四五六七八九十", "甲乙", max_length=9)
    assert len(e.ids) == 9
    v = t.vocab
    sep = e.ids.index(v["[SEP]"])
    assert sep - 1 == 4 and len(e.ids) - sep - 2 == 2      # 4 + 2 tokens survive


def test_native_matches_python(vocab):
    nt, py = ErnieTokenizer(vocab), PyErnieTokenizer(vocab)
    if not nt.native:
        pytest.skip("host library not built")
    rng = np.random.default_rng(0)
    alphabet = list("abcXYZ ,.!?é时间地点（）：12  \t") + ["​", "ß", "Ω"]
    for _ in range(200):
        a = "".join(rng.choice(alphabet, rng.integers(0, 40)))
        b = "".join(rng.choice(alphabet, rng.integers(0, 40))) if rng.random() < 0.7 else None
        ml = int(rng.choice([0, 8, 16, 64]))
        e1, e2 = py.encode(a, b, ml), nt.encode(a, b, ml)
        assert (e1.ids, e1.type_ids, e1.offsets) == (e2.ids, e2.type_ids, e2.offsets), (a, b, ml)


def test_dbc2sbc_and_split():
    assert U.dbc2sbc("ＡＢＣ，１２３") == "ABC,123"
    assert U.dbc2sbc("a　b") == "a　b"
    short, mapping = U.auto_split(["abcdefghij", "xy"], 4)
    assert short == ["abcd", "efgh", "ij", "xy"] and mapping == [[0, 1, 2], [3]]


def test_span_pairing():
    starts = [(2, 0.9), (5, 0.8), (9, 0.7)]
    ends = [(3, 0.9), (5, 0.6), (7, 0.8)]
    spans = U.pair_spans(starts, ends)
    assert [(s[0], e[0]) for s, e in spans] == [(2, 3), (5, 5)]
    assert U.pair_spans([], ends) == []


def test_auto_join_offsets_and_cls_vote():
    r = [[U.UIEResult(1, 3, 0.9, "bc")], [U.UIEResult(0, 2, 0.8, "ef")], []]
    out = U.UIEModel.auto_join(["abcd", "efgh", "ij"], [[0, 1, 2]], r)
    assert [(x.start, x.end) for x in out[0]] == [(1, 3), (4, 6)]
    c = [[U.UIEResult(0, 0, 0.6, "pos")], [U.UIEResult(0, 0, 0.9, "neg")], [U.UIEResult(0, 0, 0.5, "pos")]]
    out = U.UIEModel.auto_join(["a", "b", "c"], [[0, 1, 2]], c)
    assert out[0][0].text == "pos" and abs(out[0][0].probability - 0.55) < 1e-6


def test_uie_end_to_end_tiny(tmp_path):
    import fastdeploy_b200 as fd
    from fastdeploy_b200.models.ernie import write_ernie
    paths = write_ernie(str(tmp_path), "tiny", "uie")
    opt = fd.RuntimeOption()
    opt.use_cpu()
    m = U.UIEModel(paths["model"], paths["params"], paths["vocab"], position_prob=0.5, max_length=32,
                   schema={"person": ["age"]}, batch_size=4, runtime_option=opt, schema_language=U.SchemaLanguage.EN)
    texts = ["alice is ten years old and lives in a house by the sea " * 2, "bob"]
    res = m.predict(texts)
    assert len(res) == 2 and all(isinstance(r, dict) for r in res)
    for r in res:
        for items in r.values():
            for it in items:
                assert 0.25 < it.probability <= 1.0
                if not (it.start == 0 and it.end == 0):
                    assert texts[res.index(r)][it.start:it.end] == it.text
    d = m.predict(texts, return_dict=True)
    assert isinstance(d[0], dict)
    m.enable_padding_free(max_tokens=256, max_seqs=4, bucket_rows=64)      # same spans without padded rows
    d2 = m.predict(texts, return_dict=True)
    assert d2.keys() == d.keys() if isinstance(d, dict) else len(d2) == len(d)
    for a, b in zip(d, d2):
        assert str(a) == str(b) or _close_results(a, b)


def _close_results(a, b, tol=1e-4):
    """Two UIE result dictionaries with the same spans and probabilities within ``tol``."""
    if isinstance(a, dict):
        return a.keys() == b.keys() and all(_close_results(a[k], b[k], tol) for k in a)
    if isinstance(a, (list, tuple)):
        return len(a) == len(b) and all(_close_results(x, y, tol) for x, y in zip(a, b))
    if isinstance(a, float):
        return abs(a - b) < tol
    return a == b


def test_ernie_seq_cls_tiny(tmp_path):
    import fastdeploy_b200 as fd
    from fastdeploy_b200.models.ernie import write_ernie
    from fastdeploy_b200.text import ErnieSeqCls
    paths = write_ernie(str(tmp_path), "tiny", "seq_cls")
    opt = fd.RuntimeOption()
    opt.use_cpu()
    m = ErnieSeqCls(paths["model"], paths["params"], paths["vocab"], max_length=24, runtime_option=opt)
    out = m.predict([("the cat", "a cat sat"), "single sentence", "x"])
    assert len(out) == 3
    for k, p in out:
        assert k in (0, 1) and 0.5 <= p <= 1.0
    m.enable_padding_free(max_tokens=128, max_seqs=2, bucket_rows=32)      # 3 inputs: two packed batches
    out2 = m.predict([("the cat", "a cat sat"), "single sentence", "x"])
    assert [k for k, _ in out2] == [k for k, _ in out] and max(abs(a[1] - b[1]) for a, b in zip(out, out2)) < 1e-5


def test_packed_encoder_matches_padded_batches(tmp_path):
    """Padding-free execution (graph rewrite + interpreter): the classifier sees the same rows as the padded run."""
    import fastdeploy_b200 as fd
    from fastdeploy_b200.ir.packing import PackingError, pack_graph, pack_offsets
    from fastdeploy_b200.models.ernie import write_ernie
    from fastdeploy_b200.text.packed import PackedEncoder
    assert pack_offsets([5, 8, 9]) == ([0, 8, 16], 32)
    rng = np.random.default_rng(3)
    lens = [5, 64, 17, 100, 1]
    for task in ("seq_cls", "uie"):
        d = tmp_path / task
        write_ernie(str(d), "tiny", task, seed=1, vocab=False)
        opt = fd.RuntimeOption()
        opt.use_cpu()
        opt.set_model_path(str(d / "model.pdmodel"), str(d / "model.pdiparams"))
        rt = fd.Runtime(opt)
        names = [vi.name for vi in rt.graph.inputs]
        seqs = []
        for n in lens:
            s = [rng.integers(1, 1000, n), rng.integers(0, 2, n)]
            if task == "uie":
                s += [np.arange(n), np.ones(n, np.int64)]
            seqs.append(tuple(s))
        enc = PackedEncoder(rt, max_tokens=512, max_seqs=8, max_len=128, token_buckets=[256])
        outs = enc.infer(seqs)
        assert sorted(enc._buckets) == [256]                   # 5+64+17+100+1 tokens at aligned starts: 208 rows
        S = 128
        feeds = {n: np.zeros((len(lens), S), np.int64) for n in names}
        for i, s in enumerate(seqs):
            for n, a in zip(names, s):
                feeds[n][i, :len(a)] = a
        ref = rt.infer(feeds)
        if task == "seq_cls":
            assert outs[0].shape == ref[0].shape and np.abs(outs[0] - ref[0]).max() < 1e-5
        else:
            for k in range(2):
                for i, n in enumerate(lens):
                    assert np.abs(outs[k][i] - ref[k][i, :n]).max() < 1e-5
    with pytest.raises(ValueError):
        enc.infer([(np.zeros(200, np.int64),) * 4])           # longer than max_len
    with pytest.raises(PackingError):
        pack_graph(rt.graph, 128)                             # not optimised: no fused attention node


def test_xlm_roberta_sentencepiece_tokenizer(tmp_path):
    """A SentencePiece model trained on the spot: ids follow the XLM-R convention, offsets point into the text, and
    the SER pre-processor takes the tokenizer as it is."""
    import sentencepiece as spm
    from fastdeploy_b200.text import XLMRobertaTokenizer
    corpus = tmp_path / "corpus.txt"
    corpus.write_text("\n".join(["invoice number total amount due date", "name address phone email",
                                 "the quick brown fox jumps over the lazy dog", "total 42 invoice 2024"] * 20))
    spm.SentencePieceTrainer.train(input=str(corpus), model_prefix=str(tmp_path / "m"), vocab_size=38, model_type="unigram",
                                   character_coverage=1.0, minloglevel=2)
    tok = XLMRobertaTokenizer(str(tmp_path / "m.model"), max_length=64)
    text = "invoice total 42"
    e = tok.encode(text)
    assert e.ids[0] == 0 and e.ids[-1] == 2 and 1 not in e.ids and len(e.ids) == len(e.offsets) == len(e.attention_mask)
    assert all(i > 3 or i == 3 for i in e.ids[1:-1]) and max(e.ids) < tok.vocab_size
    pieces = tok.tokenize(text)
    assert len(pieces) == len(e.ids) - 2
    covered = "".join(text[a:b] for a, b in e.offsets[1:-1])
    assert covered.replace(" ", "") == text.replace(" ", "")
    assert tok.decode(e.ids) == text
    long = tok.encode("invoice number total amount due date " * 5, max_length=16)
    assert len(long.ids) == 16 and long.ids[-1] == 2
    pair = tok.encode("name", "address phone")
    assert pair.ids.count(2) == 3 and pair.ids[0] == 0
    from fastdeploy_b200.vision.ocr.ser import StructureV2SERViLayoutXLMPreprocessor
    pre = StructureV2SERViLayoutXLMPreprocessor(tok, max_seq_len=32)
    b = pre.run([{"bbox": [0, 0, 50, 10], "transcription": "invoice number"}], 100, 100)
    n = len(tok.encode("invoice number").ids) - 2
    assert b["segment_offset_id"] == [n] and b["input_ids"][0, 0] == 0 and b["input_ids"][0, 1 + n] == 2
