"""SentencePiece tokenizer in the XLM-RoBERTa convention (the tokenizer of LayoutXLM, which
``vision.ocr.StructureV2SERViLayoutXLM`` needs, and of the multilingual UIE models): ids of the pieces are shifted by
one so that ``<s>`` = 0, ``<pad>`` = 1, ``</s>`` = 2, ``<unk>`` = 3, and a sequence is ``<s> pieces </s>``.

The reference takes this tokenizer from external packages (``paddlenlp`` / ``paddleocr``,
python/fastdeploy/vision/ocr/ppocr/__init__.py:1142-1155); here it is a thin class over the ``sentencepiece`` model
file with character offsets for every piece.
"""
from __future__ import annotations

from typing import List, Optional, Tuple

from .tokenizer import Encoding


class XLMRobertaTokenizer:
    cls_id, pad_id, sep_id, unk_id = 0, 1, 2, 3
    _OFFSET = 1                                   # fairseq alignment: spm id k (>= 3) becomes k + 1

    def __init__(self, model_file: str, max_length: int = 512):
        import sentencepiece as spm
        self.sp = spm.SentencePieceProcessor(model_file=model_file)
        self.max_length = int(max_length)

    @property
    def vocab_size(self) -> int:
        return self.sp.get_piece_size() + self._OFFSET

    def _piece_id(self, spm_id: int) -> int:
        # sentencepiece's own 0 / 1 / 2 are <unk> / <s> / </s>; everything else moves up by one
        return self.unk_id if spm_id == self.sp.unk_id() else spm_id + self._OFFSET

    def tokenize(self, text: str) -> List[str]:
        return self.sp.encode(text, out_type=str)

    def encode(self, text: str, pair: Optional[str] = None, max_length: Optional[int] = None) -> Encoding:
        """``<s> text </s>`` (``<s> a </s></s> b </s>`` for a pair), truncated from the end of the longer part."""
        limit = max_length or self.max_length

        def pieces(t: str) -> List[Tuple[int, Tuple[int, int]]]:
            proto = self.sp.encode(t, out_type="immutable_proto")
            out = []
            for p in proto.pieces:
                out.append((self._piece_id(p.id), (p.begin, p.end)))
            return out
        a = pieces(text)
        b = pieces(pair) if pair is not None else []
        room = limit - (2 if pair is None else 4)
        while len(a) + len(b) > max(room, 0):
            if len(a) >= len(b) and a:
                a.pop()
            elif b:
                b.pop()
            else:
                break
        ids, offs, types = [self.cls_id], [(0, 0)], [0]
        for i, o in a:
            ids.append(i); offs.append(o); types.append(0)
        ids.append(self.sep_id); offs.append((0, 0)); types.append(0)
        if pair is not None:
            ids.append(self.sep_id); offs.append((0, 0)); types.append(0)
            for i, o in b:
                ids.append(i); offs.append(o); types.append(0)
            ids.append(self.sep_id); offs.append((0, 0)); types.append(0)
        enc = Encoding()
        enc.ids, enc.type_ids, enc.offsets = ids, types, offs
        enc.attention_mask = [1] * len(ids)
        return enc

    def decode(self, ids: List[int]) -> str:
        spm_ids = [i - self._OFFSET for i in ids if i > self.unk_id]
        return self.sp.decode(spm_ids)
