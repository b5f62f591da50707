"""Transformer-path ops: LayerNorm, embedding-sum + LayerNorm, masked softmax, and multi-head
attention composed from two batched tcgen05 GEMMs (csrc/kernels/transformer_ops.cu and
conv_gemm_sm100.cu in batched-weight mode).

Attention(q, k, v, mask) for ``[B, S, H*D]`` inputs runs as
  scores[b,h] = q[b,:,h,:] @ k[b,:,h,:]^T      (batched GEMM, heads = image rows of a B x H x S "image")
  p           = softmax(scale * scores + mask)  (in place, padded key columns zeroed)
  vT          = per-head transpose of v
  out[b,:,h,:] = p[b,h] @ vT[b,h]^T            (batched GEMM writing straight into [B, S, H*D])
"""
from __future__ import annotations

import ctypes
from typing import List, Optional

import torch

from .. import _native
from .base import DT_BF16, NativeOp, StatusWord, dtype_code
from .conv_gemm import ConvGemm

K_LAYERNORM, K_EMBED_LN, K_SOFTMAX, K_HEAD_TRANSPOSE = range(4)


class _TfDesc(ctypes.Structure):
    _fields_ = [("p", ctypes.c_void_p * 10), ("i", ctypes.c_longlong * 16), ("f", ctypes.c_float * 4)]


def _lib():
    lib = _native.kernels()
    if not getattr(lib, "_tf_ready", False):
        lib.fdb_transformer_create.restype = ctypes.c_void_p
        lib.fdb_transformer_create.argtypes = [ctypes.c_int, ctypes.POINTER(_TfDesc)]
        lib._tf_ready = True
    return lib


def _make(kind, ptrs, ints, floats=(), name="tf", keep=None) -> NativeOp:
    d = _TfDesc()
    for k, t in enumerate(ptrs):
        d.p[k] = (t.data_ptr() if isinstance(t, torch.Tensor) else t) if t is not None else None
    for k, v in enumerate(ints):
        d.i[k] = int(v)
    for k, v in enumerate(floats):
        d.f[k] = float(v)
    op = NativeOp(_lib().fdb_transformer_create(kind, ctypes.byref(d)), list(ptrs) + list(keep or []), name)
    op.create = ("fdb_transformer_create", kind, d)
    return op


def _bf(t) -> int:
    return 1 if dtype_code(t.dtype) == DT_BF16 else 0


def layernorm(x: torch.Tensor, y: torch.Tensor, gamma: Optional[torch.Tensor], beta: Optional[torch.Tensor], *,
              rows: int, c: int, eps: float = 1e-5, x_ld: Optional[int] = None, y_ld: Optional[int] = None,
              out_scale: float = 1.0) -> NativeOp:
    """``y = LayerNorm(x) * gamma + beta``. With an e4m3 ``y`` the result is multiplied by ``out_scale`` (the
    reciprocal of the consumer GEMM's activation scale) and stored as fp8."""
    out8 = hasattr(torch, "float8_e4m3fn") and y.dtype == torch.float8_e4m3fn
    return _make(K_LAYERNORM, [x, y, gamma, beta], [rows, c, x_ld or c, y_ld or c, _bf(x), int(out8)], [eps, out_scale],
                 "layernorm")


def embed_layernorm(ids: List[Optional[torch.Tensor]], tables: List[torch.Tensor], y: torch.Tensor,
                    gamma: torch.Tensor, beta: torch.Tensor, *, rows: int, c: int, seq: int, eps: float = 1e-5,
                    y_ld: Optional[int] = None) -> NativeOp:
    """``ids[k]`` int64 ``[rows]`` (``None`` = position index ``row % seq``), ``tables[k]`` 16-bit ``[V, c]``."""
    dev = y.device
    idp = torch.tensor([(t.data_ptr() if t is not None else 0) for t in ids] + [0] * (4 - len(ids)),
                       dtype=torch.int64, device=dev)
    tbp = torch.tensor([t.data_ptr() for t in tables] + [0] * (4 - len(tables)), dtype=torch.int64, device=dev)
    gb = torch.cat([gamma.float().reshape(-1), beta.float().reshape(-1)]).contiguous().to(dev)
    op = _make(K_EMBED_LN, [idp, tbp, y, gb], [rows, c, len(tables), seq, _bf(y), y_ld or c] +
               [int(t.shape[0]) for t in tables] + [0] * (4 - len(tables)), [eps],
               "embed_layernorm", keep=list(ids) + list(tables))
    op.pointer_tables = [idp, tbp]        # device arrays of device pointers (a plan file relocates their elements)
    return op


def masked_softmax(scores: torch.Tensor, mask: Optional[torch.Tensor], *, b: int, h: int, s: int, sk: int, ld: int,
                   scale: float, mask_b_stride: int = 0, mask_s_stride: int = 0) -> NativeOp:
    return _make(K_SOFTMAX, [scores, mask], [b, h, s, sk, ld, _bf(scores), mask_b_stride, mask_s_stride], [scale],
                 "masked_softmax")


def head_transpose(v: torch.Tensor, vt: torch.Tensor, *, b: int, s: int, h: int, d: int, v_ld: int, sp: int) -> NativeOp:
    return _make(K_HEAD_TRANSPOSE, [v, vt], [b, s, h, d, v_ld, sp], name="head_transpose")


class _AttnDesc(ctypes.Structure):
    _fields_ = [("q", ctypes.c_void_p), ("k", ctypes.c_void_p), ("vt", ctypes.c_void_p), ("out", ctypes.c_void_p),
                ("mask", ctypes.c_void_p), ("status", ctypes.c_void_p), ("seq_len", ctypes.c_void_p),
                ("seq_start", ctypes.c_void_p), ("dtype", ctypes.c_int),
                ("B", ctypes.c_int), ("H", ctypes.c_int), ("S", ctypes.c_int), ("Sk", ctypes.c_int), ("D", ctypes.c_int),
                ("q_ld", ctypes.c_int), ("k_ld", ctypes.c_int), ("o_ld", ctypes.c_int), ("skp", ctypes.c_int),
                ("total_rows", ctypes.c_int), ("m_b", ctypes.c_longlong), ("m_s", ctypes.c_longlong), ("scale", ctypes.c_float)]


def fused_attention_fits(s: int, sk: int, d: int) -> bool:
    """Whether the single-kernel attention can hold this head's K, V and probability tile on chip."""
    if d % 16 or d < 16 or d > 128 or sk > 512 or sk < 1:
        return False
    sk_pad = (sk + 15) // 16 * 16 if sk <= 256 else (sk + 31) // 32 * 32
    dch, kch = (d + 63) // 64, (sk_pad + 63) // 64
    return dch * sk_pad * 128 + kch * d * 128 + dch * 16384 + min(kch, 4) * 16384 + 1024 + 4096 <= 227 * 1024


def fused_attention_op(q, k, vt, out, mask, *, b, heads, s, sk, d, skp, scale, m_b, m_s, status, seq_len=None,
                       seq_start=None, total_rows=0) -> NativeOp:
    """One launch of csrc/kernels/attention_sm100.cu: scores and probabilities stay in tensor / shared memory.
    ``seq_len`` (int32, device, one per item) bounds each item's keys and, for self-attention, its queries;
    with ``seq_start`` (int32, device, multiples of 8) the items are packed rows of 2-D ``q``/``k``/``out``."""
    lib = _native.kernels()
    if not getattr(lib, "_attn_ready", False):
        lib.fdb_attention_create.restype = ctypes.c_void_p
        lib.fdb_attention_create.argtypes = [ctypes.POINTER(_AttnDesc)]
        if lib.fdb_attention_desc_size() != ctypes.sizeof(_AttnDesc):
            raise RuntimeError("libfdb200_kernels.so is out of date: AttnDesc layout differs")
        lib._attn_ready = True
    dd = _AttnDesc()
    dd.q, dd.k, dd.vt, dd.out = q.data_ptr(), k.data_ptr(), vt.data_ptr(), out.data_ptr()
    dd.mask = mask.data_ptr() if mask is not None else None
    dd.status = status.ptr
    dd.dtype = dtype_code(q.dtype)
    dd.B, dd.H, dd.S, dd.Sk, dd.D = b, heads, s, sk, d
    row = -2                                    # the token dimension of [B, S, C] and of packed [T, C] alike
    dd.q_ld, dd.k_ld, dd.o_ld, dd.skp = q.stride(row), k.stride(row), out.stride(row), skp
    dd.m_b, dd.m_s, dd.scale = m_b, m_s, scale
    for name, t in (("seq_len", seq_len), ("seq_start", seq_start)):
        if t is not None:
            assert t.dtype == torch.int32 and t.is_contiguous() and t.numel() >= b and t.device == q.device, name
            setattr(dd, name, t.data_ptr())
    dd.total_rows = int(total_rows)
    op = NativeOp(lib.fdb_attention_create(ctypes.byref(dd)), [q, k, vt, out, mask, status, seq_len, seq_start],
                  "attention")
    op.create = ("fdb_attention_create", None, dd)
    return op


class Attention:
    """Planned multi-head attention over fixed buffers. ``q``/``k``/``v`` are ``[B, S, H*D]`` views
    (row strides may differ, e.g. slices of a fused QKV buffer); ``out`` is ``[B, S, H*D]``."""

    def __init__(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, out: torch.Tensor, *, heads: int,
                 scale: float, mask: Optional[torch.Tensor] = None, status: Optional[StatusWord] = None,
                 fused: Optional[bool] = None, seq_lens: Optional[torch.Tensor] = None):
        b, s, hd = q.shape
        sk = k.shape[1]
        d = hd // heads
        assert d % 8 == 0, "head dim must be a multiple of 8"
        dev, dt = q.device, q.dtype
        skp = (sk + 7) // 8 * 8
        self.vt = torch.zeros(b, heads, d, skp, dtype=dt, device=dev)
        self.status = status or StatusWord(dev)
        q_ld, k_ld, v_ld, o_ld = q.stride(1), k.stride(1), v.stride(1), out.stride(1)
        rows_consecutive = (q.stride(0) == s * q_ld and k.stride(0) == sk * k_ld and v.stride(0) == sk * v_ld
                            and out.stride(0) == s * o_ld)
        can_fuse = fused_attention_fits(s, sk, d) and rows_consecutive
        if fused is None:
            fused = can_fuse
        if fused and not can_fuse:
            raise ValueError("fused attention needs <= 512 keys, a head dim that is a multiple of 16 (<= 128) and "
                             "batch items stored as consecutive rows")
        if seq_lens is not None and not fused:
            raise ValueError("per-item lengths need the fused attention kernel")
        self.fused = fused
        if fused:
            m_b = m_s = 0
            if mask is not None:
                assert mask.dtype == torch.float32
                mm = mask.reshape(b, -1, sk) if mask.numel() != b * sk else mask.reshape(b, 1, sk)
                m_b = mm.stride(0)
                m_s = mm.stride(1) if mm.shape[1] > 1 else 0
            tr = head_transpose(v, self.vt, b=b, s=sk, h=heads, d=d, v_ld=v_ld, sp=skp)
            at = fused_attention_op(q, k, self.vt, out, mask, b=b, heads=heads, s=s, sk=sk, d=d, skp=skp, scale=scale,
                                    m_b=m_b, m_s=m_s, status=self.status, seq_len=seq_lens)
            self.ops = [tr, at]
            self.keep = [q, k, v, out, mask]
            return
        self.scores = torch.zeros(b, heads, s, skp, dtype=dt, device=dev)
        # scores: "image" = B x (H rows) x (S pixels) x D channels; weights = K of the same (b, h)
        qk = ConvGemm(q, k, self.scores, in_shape=(b, heads, s, d), out_hw=(heads, s), cout=sk, x_ld=q_ld,
                      x_n_stride=q.stride(0), x_h_stride=d, y_ld=skp, status=self.status, w_batched=True,
                      w_ld=k_ld, w_h_stride=d, w_n_stride=k.stride(0), name="attn_qk")
        m_b = m_s = 0
        if mask is not None:
            assert mask.dtype == torch.float32
            mm = mask.reshape(b, -1, sk) if mask.numel() != b * sk else mask.reshape(b, 1, sk)
            m_b = mm.stride(0)
            m_s = mm.stride(1) if mm.shape[1] > 1 else 0
        sm = masked_softmax(self.scores, mask, b=b, h=heads, s=s, sk=sk, ld=skp, scale=scale, mask_b_stride=m_b,
                            mask_s_stride=m_s)
        tr = head_transpose(v, self.vt, b=b, s=sk, h=heads, d=d, v_ld=v_ld, sp=skp)
        pv = ConvGemm(self.scores, self.vt, out, in_shape=(b, heads, s, skp), out_hw=(heads, s), cout=d,
                      x_ld=skp, y_ld=o_ld, y_n_stride=out.stride(0), y_h_stride=d, status=self.status,
                      w_batched=True, w_ld=skp,
                      w_h_stride=d * skp, w_n_stride=heads * d * skp, name="attn_pv")
        self.ops = [qk, sm, tr, pv]
        self.keep = [q, k, v, out, mask]

    def launch(self, stream=None) -> None:
        for op in self.ops:
            op.launch(stream)


def pack_offsets(lengths, align: int = 8):
    """Row offsets of sequences stored back to back, each start rounded up to ``align`` rows (the attention kernel
    reads V^T by TMA, whose column coordinate must sit on a 16-byte boundary). Returns (starts, total rows)."""
    starts, at = [], 0
    for n in lengths:
        starts.append(at)
        at += (int(n) + align - 1) // align * align
    return starts, at


class PackedAttention:
    """Self-attention over padding-free batches: ``q``/``k``/``v``/``out`` are ``[T, H*D]`` views holding up to
    ``max_seqs`` sequences back to back (``seq_start[i]`` a multiple of 8, ``seq_len[i] <= max_len``). The two
    int32 device tensors are read at launch time, so one planned op (and one CUDA graph) serves every batch
    composition that fits ``T`` rows. Rows between sequences must hold finite values."""

    def __init__(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, out: torch.Tensor, *, heads: int,
                 scale: float, max_len: int, seq_start: torch.Tensor, seq_len: torch.Tensor,
                 status: Optional[StatusWord] = None):
        t, hd = q.shape
        d = hd // heads
        if not fused_attention_fits(max_len, max_len, d):
            raise ValueError("packed attention needs <= 512 tokens per sequence and a head dim that is a multiple of 16")
        assert t % 8 == 0, "the packed buffers must hold a multiple of 8 rows"
        self.status = status or StatusWord(q.device)
        self.vt = torch.zeros(1, heads, d, t, dtype=q.dtype, device=q.device)
        n = int(seq_len.numel())
        tr = head_transpose(v, self.vt, b=1, s=t, h=heads, d=d, v_ld=v.stride(0), sp=t)
        at = fused_attention_op(q, k, self.vt, out, None, b=n, heads=heads, s=max_len, sk=max_len, d=d, skp=t,
                                scale=scale, m_b=0, m_s=0, status=self.status, seq_len=seq_len, seq_start=seq_start,
                                total_rows=t)
        self.ops = [tr, at]
        self.keep = [q, k, v, out, seq_start, seq_len]

    def launch(self, stream=None) -> None:
        for op in self.ops:
            op.launch(stream)
