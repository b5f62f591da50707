"""Padding-free batches for transformer encoders: a graph rewrite.

An encoder exported for ``[B, S]`` token ids pads every sequence of a batch to the longest one; with lengths
spread over 16..512 half of the work is done on padding. Everything in such an encoder is row-wise (embedding
sum, LayerNorm, linear layers, activations) except attention, the position ids and the final pooling. This
pass turns an optimised graph into one that runs on ``[1, T]`` packed tokens (the sequences back to back, each
start a multiple of 8 rows):

* every ``Attention`` node (they must share one key-padding mask, which is dropped) becomes
  ``PackedAttention(q, k, v, seq_start, seq_len)``;
* position ids that the optimiser folded to a constant (or computed from the shape) become the graph input
  ``position_ids`` - the caller restarts them at every sequence;
* ``x[:, 0]`` pooling (``Slice`` of the first token + ``Squeeze``) becomes a row gather at ``seq_start``, so a
  classifier head sees one row per sequence; token-level outputs stay ``[1, T, ...]`` and are cut by the caller.

New graph inputs: ``position_ids`` int64 ``[1, T]``, ``seq_start`` int32 ``[N]``, ``seq_len`` int32 ``[N]``
(``N`` = most sequences per batch; unused slots have length 0). The reference has no counterpart: its back ends
run the padded graph (fastdeploy/text/uie/model.cc:565-609 pads every batch to its longest item).
"""
from __future__ import annotations

from typing import List, Sequence, Tuple

import numpy as np

from .graph import Graph, Node, ValueInfo

# operators that treat every token row independently when their other operands are per-channel constants
ROW_WISE = {"FusedGemm", "Gemm", "MatMul", "LayerNormalization", "Gelu", "Add", "Mul", "Sub", "Div", "Tanh", "Relu",
            "Sigmoid", "Erf", "Cast", "Identity", "Dropout", "Squeeze", "Unsqueeze", "Gather", "Clip", "Sqrt", "Pow",
            "Flatten"}

POSITION_IDS, SEQ_START, SEQ_LEN = "position_ids", "seq_start", "seq_len"


class PackingError(ValueError):
    pass


def pack_offsets(lengths: Sequence[int], align: int = 8) -> Tuple[List[int], int]:
    """Start row of every sequence (rounded up to ``align``) and the rows used in total."""
    starts, at = [], 0
    for n in lengths:
        starts.append(at)
        at += (int(n) + align - 1) // align * align
    return starts, at


def _is_first_token_slice(graph: Graph, node: Node) -> bool:
    if node.op != "Slice" or len(node.inputs) < 4:
        return False
    vals = [graph.initializers.get(n) for n in node.inputs[1:4]]
    if any(v is None for v in vals):
        return False
    starts, ends, axes = (np.asarray(v).reshape(-1).tolist() for v in vals)
    return starts == [0] and ends == [1] and axes == [1]


def pack_graph(graph: Graph, max_len: int) -> Graph:
    """Returns a packed copy of an optimised encoder graph (see the module text). Raises ``PackingError`` when
    the graph does not have the shape this rewrite understands."""
    g = graph.clone()
    g.toposort()
    atts = [n for n in g.nodes if n.op == "Attention"]
    if not atts:
        raise PackingError("no fused Attention node: optimise the graph with static shapes first")
    masks = {n.inputs[3] if len(n.inputs) > 3 else "" for n in atts}
    if len(masks) > 1:
        raise PackingError("the attention layers do not share one mask")
    for n in atts:
        new = Node("PackedAttention", list(n.inputs[:3]) + [SEQ_START, SEQ_LEN], list(n.outputs),
                   dict(n.attrs, max_len=int(max_len)), g.unique("n_PackedAttention"), "fdb")
        g.nodes[g.nodes.index(n)] = new
    graph_inputs = {vi.name for vi in g.inputs}
    prod = g.producers()

    def from_inputs(name: str, seen=None) -> bool:
        """Whether ``name`` depends on the values of a graph input (shape-only subgraphs were folded away)."""
        if name in graph_inputs:
            return True
        p = prod.get(name)
        if p is None:
            return False
        return any(from_inputs(i) for i in p.inputs if i)
    embeds = [n for n in g.nodes if n.op == "EmbedLayerNorm"]
    if len(embeds) != 1:
        raise PackingError("expected one fused embedding + LayerNorm at the front of the encoder")
    emb = embeds[0]
    k = emb.attr("num_tables")
    swapped = 0
    for i in range(k):
        nm = emb.inputs[i]
        if nm in g.initializers or not from_inputs(nm):
            emb.inputs[i] = POSITION_IDS
            swapped += 1
    if swapped > 1:
        raise PackingError("more than one id input of the embedding is a constant")
    if swapped == 1:
        g.inputs.append(ValueInfo(POSITION_IDS, "int64", [1, -1]))
    g.inputs.append(ValueInfo(SEQ_START, "int32", [-1]))
    g.inputs.append(ValueInfo(SEQ_LEN, "int32", [-1]))
    # first-token pooling -> one row per sequence
    cons = g.consumers()
    for n in list(g.nodes):
        if not _is_first_token_slice(g, n):
            continue
        users = cons.get(n.outputs[0], [])
        if len(users) != 1 or users[0].op != "Squeeze":
            raise PackingError("first-token slice without the squeeze that follows it in the exports known here")
        sq = users[0]
        flat = g.unique("packed_rows")                                   # [1, T, hidden] -> [T, hidden]
        g.nodes[g.nodes.index(n)] = Node("Flatten", [n.inputs[0]], [flat], {"axis": 2}, g.unique("n_Flatten"))
        g.nodes[g.nodes.index(sq)] = Node("Gather", [flat, SEQ_START], list(sq.outputs), {"axis": 0},
                                          g.unique("n_Gather"))
    g.toposort()
    g.prune()
    # what is left between the embedding and the outputs must not mix rows
    for n in g.nodes:
        if n.op in ("PackedAttention", "EmbedLayerNorm") or n.op in ROW_WISE:
            continue
        if n.op == "Slice" and len(n.inputs) >= 4 and n.inputs[3] in g.initializers and \
                np.asarray(g.initializers[n.inputs[3]]).reshape(-1).tolist() in ([-1], [2]):
            continue                      # a slice of the channels (the stacked q / k / v projection) keeps rows apart
        raise PackingError(f"operator {n.op} ({n.name}) is not known to treat token rows independently")
    g.metadata["packed"] = {"max_len": int(max_len), "position_ids": bool(swapped)}
    return g


def pack_batch(seqs: Sequence[Sequence[np.ndarray]], rows: int, max_seqs: int, pad_values: Sequence[int]):
    """``seqs[i]`` is a tuple of 1-D id arrays of one sequence (all the same length). Returns the ``[1, rows]``
    packed arrays (one per position of the tuple), position ids, starts, lengths and the start list."""
    lens = [len(s[0]) for s in seqs]
    if len(seqs) > max_seqs:
        raise ValueError(f"{len(seqs)} sequences in a plan built for {max_seqs}")
    starts, total = pack_offsets(lens)
    if total > rows:
        raise ValueError(f"{total} packed rows in a plan built for {rows}")
    n_in = len(seqs[0]) if seqs else len(pad_values)
    packed = [np.full((1, rows), int(pad_values[j]), np.int64) for j in range(n_in)]
    pos = np.zeros((1, rows), np.int64)
    for s, st, n in zip(seqs, starts, lens):
        for j in range(n_in):
            packed[j][0, st:st + n] = s[j]
        pos[0, st:st + n] = np.arange(n)
    seq_start = np.zeros(max_seqs, np.int32)
    seq_len = np.zeros(max_seqs, np.int32)
    seq_start[:len(starts)] = starts
    seq_len[:len(lens)] = lens
    return packed, pos, seq_start, seq_len, starts
