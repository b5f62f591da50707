"""Padding-free execution of an encoder model: variable-length sequences go through the network back to back.

``PackedEncoder(runtime, max_tokens, max_seqs, max_len)`` rewrites the runtime's graph with
``ir.packing.pack_graph`` and builds one plan (and CUDA graph) per bucket of packed rows; every call packs its
sequences into pinned staging arrays, copies them in, replays the plan and cuts the outputs apart again - the
sequence starts and lengths are plan inputs, so one plan serves every batch composition that fits its rows.
Sequence-level outputs (a classifier head behind first-token pooling) come back as ``[n, ...]`` arrays,
token-level outputs as one array per sequence. The reference pads instead
(fastdeploy/text/uie/model.cc:565-609, examples/text/ernie-3.0/python/seq_cls_infer.py).
"""
from __future__ import annotations

from typing import Any, Dict, List, Sequence

import numpy as np

from ..ir import packing
from ..ir.passes import optimize


class _Bucket:
    """One plan (or interpreter) for a fixed number of packed rows."""

    def __init__(self, owner: "PackedEncoder", rows: int):
        rt = owner.rt
        self.rows = rows
        shapes: Dict[str, List[int]] = {n: [1, rows] for n in owner.in_names}
        opt = optimize(rt.graph, shapes, level=2)
        self.graph = packing.pack_graph(opt, owner.max_len)
        self.has_pos = bool(self.graph.metadata["packed"]["position_ids"])
        if self.has_pos:
            shapes[packing.POSITION_IDS] = [1, rows]
        shapes[packing.SEQ_START] = [owner.max_seqs]
        shapes[packing.SEQ_LEN] = [owner.max_seqs]
        self.out_names = [vi.name for vi in self.graph.outputs]
        self.plan = None
        self.interp = None
        if rt.on_gpu:
            import torch
            from ..runtime.native_backend import build_plan
            with torch.cuda.device(rt.device):
                self.plan = build_plan(self.graph, shapes, rt.device, rt.dtype, opt_level=0)
                if rt.option.native_option.use_cuda_graph:
                    self.plan.capture()
                self.host = {n: torch.zeros(s, dtype=self.plan.inputs[n].t.dtype).pin_memory()
                             for n, s in shapes.items()}
        else:
            from ..ir.interp import Interpreter
            self.interp = Interpreter(self.graph)


class PackedEncoder:
    """``token_buckets``: the row counts plans are built for (each a multiple of 8; built on first use). A batch
    runs in the smallest bucket that holds it, because the row-wise layers cost what the bucket holds, not what
    the batch fills. Default: one bucket of ``max_tokens`` rows."""

    def __init__(self, runtime, max_tokens: int, max_seqs: int, max_len: int = 512,
                 pad_values: Sequence[int] = (), token_buckets: Sequence[int] = ()):
        buckets = sorted(set(int(b) for b in token_buckets) | {int(max_tokens)})
        if any(b % 8 or b <= 0 for b in buckets):
            raise ValueError("bucket sizes must be positive multiples of 8")
        self.rt, self.max_seqs, self.max_len = runtime, int(max_seqs), int(max_len)
        self.bucket_rows = [b for b in buckets if b <= max_tokens]
        self.in_names = [vi.name for vi in runtime.graph.inputs]
        self.pad_values = list(pad_values) + [0] * (len(self.in_names) - len(pad_values))
        self._buckets: Dict[int, _Bucket] = {}

    def bucket(self, rows_needed: int) -> _Bucket:
        for b in self.bucket_rows:
            if b >= rows_needed:
                if b not in self._buckets:
                    self._buckets[b] = _Bucket(self, b)
                return self._buckets[b]
        raise ValueError(f"{rows_needed} packed rows exceed the largest bucket ({self.bucket_rows[-1]})")

    # ------------------------------------------------------------------ packing
    def pack(self, seqs: Sequence[Sequence[np.ndarray]]):
        """Chooses the bucket and returns ``(bucket, feeds, starts, lengths)``."""
        lens = [len(s[0]) for s in seqs]
        if any(n > self.max_len for n in lens):
            raise ValueError(f"a sequence is longer than the {self.max_len} tokens this encoder was built for")
        bk = self.bucket(packing.pack_offsets(lens)[1])
        packed, pos, start, slen, starts = packing.pack_batch(seqs, bk.rows, self.max_seqs, self.pad_values)
        feeds = dict(zip(self.in_names, packed))
        if bk.has_pos:
            feeds[packing.POSITION_IDS] = pos
        feeds[packing.SEQ_START], feeds[packing.SEQ_LEN] = start, slen
        return bk, feeds, starts, lens

    @staticmethod
    def _split(arrays: List[np.ndarray], rows: int, starts: List[int], lens: List[int]) -> List[Any]:
        outs: List[Any] = []
        for a in arrays:
            if a.ndim >= 2 and a.shape[0] == 1 and a.shape[1] == rows:
                outs.append([a[0, st:st + ln] for st, ln in zip(starts, lens)])
            else:
                outs.append(a[:len(lens)])
        return outs

    # ------------------------------------------------------------------ inference
    def launch(self, bk: _Bucket, feeds: Dict[str, np.ndarray]) -> None:
        """Copies packed feeds in (through the pinned staging arrays) and replays the plan; no synchronisation."""
        for name, arr in feeds.items():
            h = bk.host[name]
            h.numpy()[...] = arr.reshape(h.shape)
            bk.plan.inputs[name].t.copy_(h, non_blocking=True)
        bk.plan.run()
        self.rt.gpu_launches += bk.plan.native_kernel_launches

    def infer(self, seqs: Sequence[Sequence[np.ndarray]]) -> List[Any]:
        bk, feeds, starts, lens = self.pack(seqs)
        if bk.interp is not None:
            res = bk.interp.run(feeds)
            arrays = [np.asarray(res[n]) for n in bk.out_names]
            return self._split(arrays, bk.rows, starts, lens)
        import torch
        with torch.cuda.device(self.rt.device):
            self.launch(bk, feeds)
            arrays = [self.rt._to_numpy(bk.plan.outputs[n].logical()) for n in bk.out_names]
            bk.plan.status.check("packed inference")
        return self._split(arrays, bk.rows, starts, lens)
