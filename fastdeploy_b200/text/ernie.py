"""ERNIE 3.0 sequence and token classification runners.

The reference has no C++ class for these: its example is ``Runtime.infer({input_ids,
token_type_ids})`` followed by a NumPy softmax (examples/text/ernie-3.0/python/seq_cls_infer.py:
tokenise with max_length padding, run, ``softmax`` + ``argmax`` + confidence). These classes pack
that recipe behind the usual model interface.
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional, Sequence, Tuple, Union

import numpy as np

from ..core.types import ModelFormat
from ..runtime.model import FastDeployModel
from ..runtime.option import RuntimeOption
from .tokenizer import ErnieTokenizer


def softmax(x: np.ndarray, axis: int = -1) -> np.ndarray:
    m = x.max(axis=axis, keepdims=True)
    e = np.exp(x - m)
    return e / e.sum(axis=axis, keepdims=True)


class _ErnieBase(FastDeployModel):
    def __init__(self, model_file: str, params_file: str, vocab_file: str, max_length: int = 128,
                 runtime_option: Optional[RuntimeOption] = None, model_format: int = ModelFormat.PADDLE):
        super().__init__(runtime_option)
        self.runtime_option.set_model_path(model_file, params_file, model_format)
        self.max_length = max_length
        self.tokenizer = ErnieTokenizer(vocab_file)
        self.tokenizer.enable_truncation(max_length)
        self.init_runtime()

    def enable_padding_free(self, max_tokens: int = 16384, max_seqs: int = 64, bucket_rows: int = 2048) -> None:
        """Runs batches without padding (text/packed.py): sequences back to back in plans of ``bucket_rows`` steps
        up to ``max_tokens`` rows, at most ``max_seqs`` sequences per batch. Results are those of the padded run."""
        from .packed import PackedEncoder
        self._packed = PackedEncoder(self.runtime, max_tokens, max_seqs, self.max_length,
                                     pad_values=[self.tokenizer.pad_id, 0],
                                     token_buckets=range(bucket_rows, max_tokens + 1, bucket_rows))

    def _logits(self, encs, feed) -> List[np.ndarray]:
        """Per-sequence logits of the first output: through the packed plans when enabled, else the padded batch."""
        packed = getattr(self, "_packed", None)
        if packed is None:
            return list(np.asarray(self.runtime.infer(feed)[0], dtype=np.float32))
        arrays = list(feed.values())
        out: List[np.ndarray] = []
        for s in range(0, len(encs), packed.max_seqs):
            seqs = []
            for i in range(s, min(s + packed.max_seqs, len(encs))):
                n = int(sum(encs[i].attention_mask))
                seqs.append(tuple(a[i, :n] for a in arrays))
            res = packed.infer(seqs)[0]
            out += [np.asarray(r, np.float32) for r in res]
        return out

    def encode(self, texts: Sequence[Union[str, Tuple[str, str]]], pad_to_max: bool = False):
        encs = self.tokenizer.encode_batch(list(texts), pad=True)
        if pad_to_max:
            for e in encs:
                e.pad(self.max_length, self.tokenizer.pad_id)
        ids = np.asarray([e.ids for e in encs], dtype=np.int64)
        types = np.asarray([e.type_ids for e in encs], dtype=np.int64)
        names = [i.name for i in self.runtime.get_input_infos()]
        return encs, dict(zip(names, [ids, types]))


class ErnieSeqCls(_ErnieBase):
    """Sentence (pair) classification: returns ``(label, confidence)`` per input."""

    def predict(self, texts: Sequence[Union[str, Tuple[str, str]]], batch_size: int = 32) -> List[Tuple[int, float]]:
        out: List[Tuple[int, float]] = []
        for s in range(0, len(texts), batch_size):
            encs, feed = self.encode(texts[s:s + batch_size])
            logits = np.stack(self._logits(encs, feed))
            probs = softmax(logits.reshape(logits.shape[0], -1))
            for row in probs:
                k = int(row.argmax())
                out.append((k, float(row[k])))
        return out


class ErnieTokenCls(_ErnieBase):
    """Token classification: per input a list of ``(label, confidence, (char_start, char_end))`` for
    the tokens of the first segment (special tokens are skipped)."""

    def predict(self, texts: Sequence[str], batch_size: int = 32):
        out = []
        for s in range(0, len(texts), batch_size):
            encs, feed = self.encode(texts[s:s + batch_size])
            probs = [softmax(l, axis=-1) for l in self._logits(encs, feed)]     # packed rows stop at the real length
            for e, p in zip(encs, probs):
                row = []
                for t, (off, m) in enumerate(zip(e.offsets, e.attention_mask)):
                    if m == 0 or off == (0, 0):
                        continue
                    k = int(p[t].argmax())
                    row.append((k, float(p[t, k]), off))
                out.append(row)
        return out
