"""Universal Information Extraction over an ERNIE encoder.

Behaviour follows fastdeploy/text/uie/model.cc (schema tree walked breadth first :722-800,
prompt construction and long-text splitting :487-545 / :253-300, candidate thresholding and
span pairing :302-347, span -> text conversion :349-412, joining of split texts :414-485,
child prompt prefixes :638-658, full-width folding of prompts :31-56) and the Python wrapper
python/fastdeploy/text/uie/__init__.py:22-95.

The encoder runs through :class:`fastdeploy_b200.Runtime` (inputs ``input_ids, token_type_ids,
position_ids, attention_mask`` as int64 ``[B, S]``, outputs start / end probabilities ``[B, S]``).
"""
from __future__ import annotations

from collections import deque
from typing import Any, Dict, List, Optional, Sequence, Tuple, Union

import numpy as np

from ..core.types import ModelFormat
from ..runtime.model import FastDeployModel
from ..runtime.option import RuntimeOption
from .tokenizer import Encoding, ErnieTokenizer


class SchemaLanguage:
    ZH = 0
    EN = 1


class SchemaNode:
    """One node of the extraction schema; ``children`` may be names, nodes, lists or dicts."""

    def __init__(self, name: str, children: Any = None):
        self.name = name
        self.children: List["SchemaNode"] = []
        self.prefix: List[List[str]] = []
        self.relations: List[List["UIEResult"]] = []
        for c in _as_nodes(children):
            self.children.append(c)

    def add_child(self, child: Union[str, "SchemaNode"]) -> None:
        self.children.append(child if isinstance(child, SchemaNode) else SchemaNode(child))


def _as_nodes(spec: Any) -> List[SchemaNode]:
    if spec is None or spec == []:
        return []
    if isinstance(spec, SchemaNode):
        return [spec]
    if isinstance(spec, str):
        return [SchemaNode(spec)]
    if isinstance(spec, dict):
        return [SchemaNode(k, v) for k, v in spec.items()]
    out: List[SchemaNode] = []
    for item in spec:
        out.extend(_as_nodes(item))
    return out


class UIEResult:
    def __init__(self, start: int = 0, end: int = 0, probability: float = 0.0, text: str = ""):
        self.start, self.end, self.probability, self.text = start, end, probability, text
        self.relation: Dict[str, List["UIEResult"]] = {}

    def get_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {"text": self.text, "probability": self.probability}
        if not (self.start == 0 and self.end == 0):
            d["start"], d["end"] = self.start, self.end
        if self.relation:
            d["relation"] = {k: [r.get_dict() for r in v] for k, v in self.relation.items()}
        return d

    def __repr__(self) -> str:
        return f"UIEResult({self.get_dict()})"


def dbc2sbc(s: str) -> str:
    """Full-width ASCII variants (U+FF01..U+FF5E) become ASCII; everything else is kept, the
    ideographic space included (fastdeploy/text/uie/model.cc:31-56)."""
    out = []
    for ch in s:
        c = ord(ch)
        folded = 0x20 if c == 0x3000 else c - 0xFEE0
        out.append(chr(folded) if 0x21 <= folded <= 0x7E else ch)
    return "".join(out)


def auto_split(texts: Sequence[str], max_length: int) -> Tuple[List[str], List[List[int]]]:
    """Cuts every text into pieces of at most ``max_length`` code points; returns the pieces and,
    per input text, the indices of its pieces."""
    short: List[str] = []
    mapping: List[List[int]] = []
    for t in texts:
        if len(t) <= max_length:
            mapping.append([len(short)])
            short.append(t)
        else:
            ids = []
            for s in range(0, len(t), max_length):
                ids.append(len(short))
                short.append(t[s:s + max_length])
            mapping.append(ids)
    return short, mapping


def candidates(prob_row: np.ndarray, threshold: float) -> List[Tuple[int, float]]:
    idx = np.nonzero(prob_row > threshold)[0]
    return [(int(i), float(prob_row[i])) for i in idx]


def pair_spans(starts: List[Tuple[int, float]], ends: List[Tuple[int, float]]):
    """Two-pointer sweep over the sorted start and end candidates (model.cc:325-347); the result is
    ordered by (start, end) and free of duplicates."""
    spans = set()
    i = j = 0
    while i < len(starts) and j < len(ends):
        s, e = starts[i], ends[j]
        if s[0] == e[0]:
            spans.add((s, e))
            i += 1
            j += 1
        elif s[0] < e[0]:
            spans.add((s, e))
            i += 1
        else:
            j += 1
    return sorted(spans, key=lambda se: (se[0][0], se[1][0]))


class UIEModel(FastDeployModel):
    def __init__(self, model_file: str, params_file: str, vocab_file: str, position_prob: float = 0.5,
                 max_length: int = 128, schema: Any = None, batch_size: int = 64,
                 runtime_option: Optional[RuntimeOption] = None, model_format: int = ModelFormat.PADDLE,
                 schema_language: int = SchemaLanguage.ZH):
        super().__init__(runtime_option)
        self.runtime_option.set_model_path(model_file, params_file, model_format)
        self.position_prob = position_prob
        self.max_length = max_length
        self.batch_size = batch_size
        self.schema_language = schema_language
        self.tokenizer = ErnieTokenizer(vocab_file)
        self.tokenizer.enable_truncation(max_length)
        self.init_runtime()
        self.root = SchemaNode("root")
        self.set_schema(schema if schema is not None else [])

    def model_name(self) -> str:
        return "UIEModel"

    def set_schema(self, schema: Any) -> None:
        self.root = SchemaNode("root", schema)

    # ------------------------------------------------------------------ stages
    def construct_texts_and_prompts(self, raw_texts: Sequence[str], node: SchemaNode):
        texts: List[str] = []
        prompts: List[str] = []
        map_raw: List[List[int]] = []
        if not node.prefix:
            for i, t in enumerate(raw_texts):
                texts.append(t)
                prompts.append(dbc2sbc(node.name))
                map_raw.append([i])
        else:
            idx = 0
            for i, t in enumerate(raw_texts):
                pres = node.prefix[i]
                for pre in pres:
                    texts.append(t)
                    prompts.append(dbc2sbc(pre + node.name))
                map_raw.append(list(range(idx, idx + len(pres))))
                idx += len(pres)
        if not prompts:
            return None
        max_prompt = max(len(p) for p in prompts)
        short, mapping = auto_split(texts, self.max_length - 3 - max_prompt)
        short_prompts: List[str] = []
        for i, ids in enumerate(mapping):
            short_prompts.extend([prompts[i]] * len(ids))
        return short, short_prompts, map_raw, mapping

    def preprocess(self, texts: Sequence[str], prompts: Sequence[str]):
        encs = self.tokenizer.encode_batch(list(zip(prompts, texts)), pad=True)
        seq = len(encs[0].ids)
        n = len(encs)
        ids = np.asarray([e.ids for e in encs], dtype=np.int64).reshape(n, seq)
        types = np.asarray([e.type_ids for e in encs], dtype=np.int64).reshape(n, seq)
        mask = np.asarray([e.attention_mask for e in encs], dtype=np.int64).reshape(n, seq)
        pos = np.tile(np.arange(seq, dtype=np.int64), (n, 1))
        # the four inputs are bound by position, as the reference does (model.cc:567-599)
        names = [i.name for i in self.runtime.get_input_infos()]
        return encs, dict(zip(names, [ids, types, pos, mask]))

    def postprocess(self, start_prob: np.ndarray, end_prob: np.ndarray, encs: List[Encoding], texts: Sequence[str],
                    prompts: Sequence[str], mapping: List[List[int]]) -> List[List[UIEResult]]:
        per_short: List[List[UIEResult]] = []
        for i, e in enumerate(encs):
            spans = pair_spans(candidates(start_prob[i], self.position_prob), candidates(end_prob[i], self.position_prob))
            offs = e.offsets
            first_sep = next((k for k in range(1, len(offs)) if offs[k] == (0, 0)), len(offs))
            prompt_end_tok = first_sep - 1
            res: List[UIEResult] = []
            for (s_tok, s_p), (e_tok, e_p) in spans:
                start, end = offs[s_tok][0], offs[e_tok][1]
                if 0 < e_tok <= prompt_end_tok:      # the span lies in the prompt: a classification answer
                    res.append(UIEResult(0, 0, s_p * e_p, prompts[i][start:end]))
                else:
                    res.append(UIEResult(start, end, s_p * e_p, texts[i][start:end]))
            per_short.append(res)
        return self.auto_join(texts, mapping, per_short)

    @staticmethod
    def auto_join(short_texts: Sequence[str], mapping: List[List[int]], results: List[List[UIEResult]]):
        first = next((r for r in results if r), None)
        is_cls = first is not None and first[0].start == 0 and first[0].end == 0
        final: List[List[UIEResult]] = []
        if is_cls:
            for ids in mapping:
                votes: Dict[str, List[float]] = {}
                for k in ids:
                    if results[k]:
                        votes.setdefault(results[k][0].text, []).append(results[k][0].probability)
                out: List[UIEResult] = []
                if votes:
                    best = max(votes.items(), key=lambda kv: sum(kv[1]))
                    out.append(UIEResult(0, 0, sum(best[1]) / len(best[1]), best[0]))
                final.append(out)
        else:
            for ids in mapping:
                off = 0
                out = []
                for k in ids:
                    for r in results[k]:
                        r.start += off
                        r.end += off
                    out.extend(results[k])
                    off += len(short_texts[k])
                final.append(out)
        return final

    def enable_padding_free(self, max_tokens: int = 16384, max_seqs: int = 64, bucket_rows: int = 2048) -> None:
        """Runs the prompt + text batches without padding (text/packed.py); probabilities past a sequence's end,
        which the padded run computes and the decoder ignores, come back as zero."""
        from .packed import PackedEncoder
        self._packed = PackedEncoder(self.runtime, max_tokens, max_seqs, self.max_length,
                                     token_buckets=range(bucket_rows, max_tokens + 1, bucket_rows))

    def _infer_batched(self, feed: Dict[str, np.ndarray]) -> Tuple[np.ndarray, np.ndarray]:
        first = next(iter(feed.values()))
        n = first.shape[0]
        starts, ends = [], []
        packed = getattr(self, "_packed", None)
        if packed is not None:
            arrays = list(feed.values())
            lens = arrays[3].sum(axis=1).astype(np.int64)               # the attention mask is the fourth input
            sp, ep = np.zeros(first.shape, np.float32), np.zeros(first.shape, np.float32)
            for s in range(0, n, packed.max_seqs):
                idx = range(s, min(s + packed.max_seqs, n))
                outs = packed.infer([tuple(a[i, :lens[i]] for a in arrays) for i in idx])
                for j, i in enumerate(idx):
                    sp[i, :lens[i]] = np.asarray(outs[0][j]).reshape(-1)
                    ep[i, :lens[i]] = np.asarray(outs[1][j]).reshape(-1)
            return sp, ep
        for s in range(0, n, self.batch_size):
            chunk = {k: v[s:s + self.batch_size] for k, v in feed.items()}
            shape = next(iter(chunk.values())).shape
            outs = self.runtime.infer(chunk)
            starts.append(np.asarray(outs[0], dtype=np.float32).reshape(shape))
            ends.append(np.asarray(outs[1], dtype=np.float32).reshape(shape))
        return np.concatenate(starts), np.concatenate(ends)

    # ------------------------------------------------------------------ API
    def predict(self, texts: Sequence[str], return_dict: bool = False):
        texts = list(texts)
        results: List[Dict[str, List[UIEResult]]] = [dict() for _ in texts]
        queue = deque(self.root.children)
        for n in queue:
            n.prefix, n.relations = [], []
        while queue:
            node = queue.popleft()
            built = self.construct_texts_and_prompts(texts, node)
            results_list: List[List[UIEResult]] = []
            map_raw: List[List[int]] = [[] for _ in texts]
            if built is not None:
                short, short_prompts, map_raw, mapping = built
                encs, feed = self.preprocess(short, short_prompts)
                sp, ep = self._infer_batched(feed)
                results_list = self.postprocess(sp, ep, encs, short, short_prompts, mapping)
            new_rel: List[List[UIEResult]] = [[] for _ in texts]
            if not node.relations:
                for i, ids in enumerate(map_raw):
                    for k in ids:
                        if results_list[k]:
                            results[i].setdefault(node.name, []).extend(results_list[k])
                    new_rel[i] = list(results[i].get(node.name, []))
            else:
                for i, ids in enumerate(map_raw):
                    for j, k in enumerate(ids):
                        if results_list[k]:
                            node.relations[i][j].relation.setdefault(node.name, []).extend(results_list[k])
                for i, rels in enumerate(node.relations):
                    for r in rels:
                        new_rel[i].extend(r.relation.get(node.name, []))
            prefix: List[List[str]] = [[] for _ in texts]
            for i, ids in enumerate(map_raw):
                for k in ids:
                    for r in results_list[k]:
                        prefix[i].append(r.text + "的" if self.schema_language == SchemaLanguage.ZH
                                         else " of " + r.text)
            for child in node.children:
                child.relations = new_rel
                child.prefix = prefix
                queue.append(child)
        if not return_dict:
            return results
        return [{k: [r.get_dict() for r in v] for k, v in res.items()} for res in results]
