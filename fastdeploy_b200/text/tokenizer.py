"""ERNIE / BERT WordPiece tokenizer.

The reference links PaddleNLP's external ``fast_tokenizer`` library
(``ErnieFastTokenizer``, used from fastdeploy/text/uie/model.cc:177-184, 557-622). This module
provides the same behaviour twice: :class:`ErnieTokenizer` drives the C++ implementation in
csrc/cpu/tokenizer.cc through ctypes, :class:`PyErnieTokenizer` is a pure-Python mirror with
identical character classes that serves as the test oracle and as the fallback when the host
library has not been built.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple, Union

import numpy as np

from .. import _native

SPECIAL_TOKENS = ["[PAD]", "[CLS]", "[SEP]", "[UNK]", "[MASK]"]


@dataclass
class Encoding:
    """One encoded (pair of) segment(s); offsets are code-point ranges relative to each segment."""
    ids: List[int] = field(default_factory=list)
    type_ids: List[int] = field(default_factory=list)
    attention_mask: List[int] = field(default_factory=list)
    offsets: List[Tuple[int, int]] = field(default_factory=list)

    def pad(self, length: int, pad_id: int) -> None:
        extra = length - len(self.ids)
        if extra > 0:
            self.ids += [pad_id] * extra
            self.type_ids += [0] * extra
            self.attention_mask += [0] * extra
            self.offsets += [(0, 0)] * extra


# ------------------------------------------------------------------ character classes (mirrored in C++)
def _is_whitespace(c: int) -> bool:
    return c in (0x20, 0x09, 0x0A, 0x0D, 0xA0, 0x1680, 0x202F, 0x205F, 0x3000) or 0x2000 <= c <= 0x200A


def _is_control(c: int) -> bool:
    if c in (0x09, 0x0A, 0x0D):
        return False
    return (c < 0x20 or 0x7F <= c < 0xA0 or c == 0xAD or 0x200B <= c <= 0x200F or 0x202A <= c <= 0x202E
            or 0x2060 <= c <= 0x2064 or c == 0xFEFF)


def _is_cjk(c: int) -> bool:
    return (0x4E00 <= c <= 0x9FFF or 0x3400 <= c <= 0x4DBF or 0x20000 <= c <= 0x2A6DF or 0x2A700 <= c <= 0x2B73F
            or 0x2B740 <= c <= 0x2B81F or 0x2B820 <= c <= 0x2CEAF or 0xF900 <= c <= 0xFAFF or 0x2F800 <= c <= 0x2FA1F)


def _is_punct(c: int) -> bool:
    if 33 <= c <= 47 or 58 <= c <= 64 or 91 <= c <= 96 or 123 <= c <= 126:
        return True
    if c in (0xA1, 0xA7, 0xAB, 0xB6, 0xB7, 0xBB, 0xBF):
        return True
    return (0x2010 <= c <= 0x2027 or 0x2030 <= c <= 0x205E or 0x3001 <= c <= 0x303F or 0xFF01 <= c <= 0xFF0F
            or 0xFF1A <= c <= 0xFF20 or 0xFF3B <= c <= 0xFF40 or 0xFF5B <= c <= 0xFF65)


_LATIN1_BASE = "aaaaaa\0ceeeeiiii\0nooooo\0\0uuuuy\0y"


def _fold(c: int) -> int:
    if 0x41 <= c <= 0x5A:
        return c + 32
    if 0xC0 <= c <= 0xDE and c != 0xD7:
        c += 0x20
    if 0x391 <= c <= 0x3A9 and c != 0x3A2:
        return c + 0x20
    if 0x410 <= c <= 0x42F:
        return c + 0x20
    if 0x400 <= c <= 0x40F:
        return c + 0x50
    if 0xE0 <= c <= 0xFF:
        b = _LATIN1_BASE[c - 0xE0]
        if b != "\0":
            return ord(b)
    return c


def load_vocab(path: str) -> Dict[str, int]:
    vocab: Dict[str, int] = {}
    with open(path, encoding="utf-8") as f:
        for i, line in enumerate(f):
            vocab[line.rstrip("\r\n")] = i
    return vocab


class PyErnieTokenizer:
    """Pure-Python implementation (oracle / fallback)."""

    def __init__(self, vocab_file: str, do_lower_case: bool = True):
        self.vocab = load_vocab(vocab_file)
        self.do_lower_case = do_lower_case
        self.pad_id = self.vocab.get("[PAD]", 0)
        self.unk_id = self.vocab.get("[UNK]", 0)
        self.cls_id = self.vocab.get("[CLS]", 0)
        self.sep_id = self.vocab.get("[SEP]", 0)
        self.max_length = 0

    def enable_truncation(self, max_length: int) -> None:
        """Longest-first truncation from the right (fastdeploy/text/uie/model.cc:182-184)."""
        self.max_length = max_length

    def _wordpiece(self, word: List[int], pos: List[int], out: List[Tuple[int, int, int]]) -> None:
        n = len(word)
        if n > 100:
            out.append((self.unk_id, pos[0], pos[-1] + 1))
            return
        pieces = []
        start = 0
        while start < n:
            end, found = n, -1
            while start < end:
                s = ("##" if start > 0 else "") + "".join(chr(c) for c in word[start:end])
                if s in self.vocab:
                    found = self.vocab[s]
                    break
                end -= 1
            if found < 0:
                out.append((self.unk_id, pos[0], pos[-1] + 1))
                return
            pieces.append((found, pos[start], pos[end - 1] + 1))
            start = end
        out.extend(pieces)

    def encode_segment(self, text: str) -> List[Tuple[int, int, int]]:
        out: List[Tuple[int, int, int]] = []
        word: List[int] = []
        pos: List[int] = []

        def flush():
            if word:
                self._wordpiece(word, pos, out)
            word.clear()
            pos.clear()

        for i, ch in enumerate(text):
            c = ord(ch)
            if c == 0 or c == 0xFFFD or _is_control(c):
                continue
            if _is_whitespace(c):
                flush()
                continue
            f = _fold(c) if self.do_lower_case else c
            if _is_cjk(c) or _is_punct(c):
                flush()
                word.append(f)
                pos.append(i)
                flush()
                continue
            word.append(f)
            pos.append(i)
        flush()
        return out

    def encode(self, text: str, pair: Optional[str] = None, max_length: Optional[int] = None) -> Encoding:
        pa = self.encode_segment(text)
        pb = self.encode_segment(pair) if pair is not None else []
        specials = 3 if pair is not None else 2
        ml = self.max_length if max_length is None else max_length
        if ml and ml > 0:
            over = len(pa) + len(pb) + specials - ml
            while over > 0 and (pa or pb):
                if len(pa) > len(pb):
                    pa.pop()
                elif pb:
                    pb.pop()
                else:
                    pa.pop()
                over -= 1
        e = Encoding()

        def put(i, t, s, en):
            e.ids.append(i)
            e.type_ids.append(t)
            e.attention_mask.append(1)
            e.offsets.append((s, en))

        put(self.cls_id, 0, 0, 0)
        for i, s, en in pa:
            put(i, 0, s, en)
        put(self.sep_id, 0, 0, 0)
        if pair is not None:
            for i, s, en in pb:
                put(i, 1, s, en)
            put(self.sep_id, 1, 0, 0)
        return e

    def encode_batch(self, items: Sequence[Union[str, Tuple[str, str]]], pad: bool = True) -> List[Encoding]:
        encs = [self.encode(*((it, None) if isinstance(it, str) else it)) for it in items]
        if pad and encs:
            longest = max(len(e.ids) for e in encs)
            for e in encs:
                e.pad(longest, self.pad_id)
        return encs


class ErnieTokenizer(PyErnieTokenizer):
    """Tokenizer backed by the C++ implementation; same interface as :class:`PyErnieTokenizer`."""

    def __init__(self, vocab_file: str, do_lower_case: bool = True):
        super().__init__(vocab_file, do_lower_case)
        self._h = None
        if _native.cpu_available():
            lib = _native.cpu()
            lib.fdb_tok_create.restype = ctypes.c_void_p
            lib.fdb_tok_create.argtypes = [ctypes.c_char_p, ctypes.c_int]
            lib.fdb_tok_destroy.argtypes = [ctypes.c_void_p]
            lib.fdb_tok_encode_pair.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_char_p, ctypes.c_int] + \
                [ctypes.POINTER(ctypes.c_int)] * 4 + [ctypes.c_int]
            self._lib = lib
            self._h = lib.fdb_tok_create(vocab_file.encode(), int(do_lower_case))
            if not self._h:
                raise RuntimeError("tokenizer: cannot read " + vocab_file)

    @property
    def native(self) -> bool:
        return self._h is not None

    def encode(self, text: str, pair: Optional[str] = None, max_length: Optional[int] = None) -> Encoding:
        if self._h is None or "\0" in text or (pair is not None and "\0" in pair):
            return super().encode(text, pair, max_length)
        ml = self.max_length if max_length is None else max_length
        cap = len(text) + (len(pair) if pair is not None else 0) + 3
        if ml and ml > 0:
            cap = min(cap, ml)
        cap = max(cap, 3)
        arr = (ctypes.c_int * (4 * cap))()
        ptrs = [ctypes.cast(ctypes.byref(arr, 4 * cap * k), ctypes.POINTER(ctypes.c_int)) for k in range(4)]
        n = self._lib.fdb_tok_encode_pair(self._h, text.encode("utf-8"), pair.encode("utf-8") if pair is not None else None,
                                          int(ml or 0), ptrs[0], ptrs[1], ptrs[2], ptrs[3], cap)
        a = np.frombuffer(arr, dtype=np.int32).reshape(4, cap)[:, :n]
        e = Encoding()
        e.ids = a[0].tolist()
        e.type_ids = a[1].tolist()
        e.attention_mask = [1] * n
        e.offsets = list(zip(a[2].tolist(), a[3].tolist()))
        return e

    def __del__(self):
        try:
            if self._h:
                self._lib.fdb_tok_destroy(self._h)
        except Exception:
            pass


def write_synthetic_vocab(path: str, size: int, seed: int = 0) -> List[str]:
    """Writes a deterministic ``vocab.txt`` of ``size`` entries: the special tokens, ASCII letters,
    digits and punctuation, common CJK characters, two- and three-letter word starts and ``##``
    continuations. Enough structure for WordPiece to split arbitrary Latin / CJK text without
    falling back to ``[UNK]`` all the time; there is no network access for a real vocabulary."""
    toks: List[str] = list(SPECIAL_TOKENS)
    seen = set(toks)

    def add(t: str) -> None:
        if t not in seen and len(toks) < size:
            seen.add(t)
            toks.append(t)

    for c in "abcdefghijklmnopqrstuvwxyz0123456789":
        add(c)
    for c in "abcdefghijklmnopqrstuvwxyz0123456789":
        add("##" + c)
    for c in "!\"#$%&'()*+,-./:;<=>?@[\\]^_`{|}~，。、；：？！（）《》“”‘’":
        add(c)
    for cp in range(0x4E00, 0x4E00 + max(0, min(0x9FFF - 0x4E00 + 1, size // 2))):
        add(chr(cp))
    rng = np.random.default_rng(seed)
    letters = "etaoinshrdlcumwfgypbvkjxqz"
    common = ["the", "of", "and", "to", "in", "is", "for", "that", "on", "with", "as", "was", "by", "at", "from",
              "ing", "ed", "er", "es", "ly", "tion", "ment", "ness", "al", "ic", "ous", "ive", "able"]
    for w in common:
        add(w)
        add("##" + w)
    while len(toks) < size:
        n = int(rng.integers(2, 5))
        w = "".join(letters[int(i)] for i in np.minimum(rng.geometric(0.12, n) - 1, 25))
        add(w if rng.random() < 0.5 else "##" + w)
    with open(path, "w", encoding="utf-8") as f:
        f.write("\n".join(toks) + "\n")
    return toks
