"""tcgen05 implicit-GEMM convolution / GEMM (csrc/kernels/conv_gemm_sm100.cu).

Activations are NHWC fp16/bf16; weights are packed ``[Cout, KH*KW*cin_pad]``
(K-major, ``cin_pad`` = Cin rounded up to 64). A GEMM ``y[M,N] = x[M,K] @ w[N,K]^T``
is the 1x1 case over a ``1 x M`` image. This is the op the reference hands to
TensorRT / Paddle Inference / ONNX Runtime
(fastdeploy/runtime/backends/tensorrt/trt_backend.cc:347).
"""
from __future__ import annotations

import ctypes
from typing import Sequence, Optional, Tuple

import torch

from .. import _native
from .base import ACT, NativeOp, StatusWord, dtype_code

K_BLOCK = 64


class _ConvGemmDesc(ctypes.Structure):
    _fields_ = [
        ("x", ctypes.c_void_p), ("w", ctypes.c_void_p), ("bias", ctypes.c_void_p),
        ("residual", ctypes.c_void_p), ("y", ctypes.c_void_p), ("status", ctypes.c_void_p),
        ("dtype", ctypes.c_int), ("out_dtype", ctypes.c_int),
        ("N", ctypes.c_int), ("H", ctypes.c_int), ("W", ctypes.c_int), ("Cin", ctypes.c_int), ("x_ld", ctypes.c_int),
        ("Ho", ctypes.c_int), ("Wo", ctypes.c_int), ("Cout", ctypes.c_int), ("y_ld", ctypes.c_int),
        ("KH", ctypes.c_int), ("KW", ctypes.c_int), ("stride", ctypes.c_int), ("pad_h", ctypes.c_int),
        ("pad_w", ctypes.c_int),
        ("res_ld", ctypes.c_int), ("res_mode", ctypes.c_int),
        ("act", ctypes.c_int), ("act_alpha", ctypes.c_float), ("act_beta", ctypes.c_float),
        ("tile_w", ctypes.c_int), ("tile_h", ctypes.c_int), ("block_n", ctypes.c_int), ("max_ctas", ctypes.c_int),
        ("x_n_stride", ctypes.c_longlong), ("y_n_stride", ctypes.c_longlong), ("res_n_stride", ctypes.c_longlong),
        ("halo_mode", ctypes.c_int),
        ("w_batched", ctypes.c_int), ("w_ld", ctypes.c_int), ("w_h_stride", ctypes.c_longlong),
        ("w_n_stride", ctypes.c_longlong),
        ("x_h_stride", ctypes.c_longlong), ("y_h_stride", ctypes.c_longlong), ("res_h_stride", ctypes.c_longlong),
        ("y_tma_mode", ctypes.c_int),
        ("trace", ctypes.c_void_p),
        ("peer_mode", ctypes.c_int), ("peer_rows", ctypes.c_int), ("peer_rank", ctypes.c_int),
        ("peer_world", ctypes.c_int),
        ("peer_ptrs", ctypes.c_void_p * 8), ("peer_counters", ctypes.c_void_p * 8),
        ("peer_ready", ctypes.c_void_p), ("peer_copiers", ctypes.c_int),
        ("scale_a", ctypes.c_void_p), ("scale_b", ctypes.c_void_p),
        ("pair_mode", ctypes.c_int), ("out_scale", ctypes.c_float),
    ]


def _lib():
    lib = _native.kernels()
    if not getattr(lib, "_conv_gemm_ready", False):
        lib.fdb_conv_gemm_create.restype = ctypes.c_void_p
        lib.fdb_conv_gemm_create.argtypes = [ctypes.POINTER(_ConvGemmDesc)]
        lib.fdb_conv_gemm_info.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_int)]
        lib.fdb_conv_gemm_variant.argtypes = [ctypes.c_void_p]
        if lib.fdb_conv_gemm_desc_size() != ctypes.sizeof(_ConvGemmDesc):
            raise RuntimeError("libfdb200_kernels.so is out of date: ConvGemmDesc layout differs; rebuild with "
                               "`python -m fastdeploy_b200._native.build`")
        lib._conv_gemm_ready = True
    return lib


def pack_conv_weight(w: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """``[Cout, Cin, KH, KW]`` -> ``[Cout, KH*KW*cin_pad]`` with zero-padded channels."""
    cout, cin, kh, kw = w.shape
    cin_pad = (cin + K_BLOCK - 1) // K_BLOCK * K_BLOCK
    out = torch.zeros(cout, kh, kw, cin_pad, dtype=dtype, device=w.device)
    out[..., :cin] = w.permute(0, 2, 3, 1).to(dtype)
    return out.reshape(cout, kh * kw * cin_pad).contiguous()


def pack_linear_weight(w: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """``[N, K]`` (torch Linear layout) -> K padded to a multiple of 64."""
    n, k = w.shape
    return pack_conv_weight(w.reshape(n, k, 1, 1), dtype)


class ConvGemm(NativeOp):
    """One planned convolution launch. All tensors are fixed at construction."""

    def __init__(self, x: torch.Tensor, w_packed: torch.Tensor, y: torch.Tensor, *,
                 in_shape: Tuple[int, int, int, int], out_hw: Tuple[int, int], cout: int,
                 kernel: Tuple[int, int] = (1, 1), stride: int = 1, pad: Tuple[int, int] = (0, 0),
                 bias: Optional[torch.Tensor] = None, residual: Optional[torch.Tensor] = None,
                 res_mode: int = 0, act: Optional[str] = None, act_alpha: float = 0.0, act_beta: float = 0.0,
                 x_ld: Optional[int] = None, y_ld: Optional[int] = None, res_ld: Optional[int] = None,
                 status: Optional[StatusWord] = None, tile: Tuple[int, int] = (0, 0), block_n: int = 0,
                 max_ctas: int = 0, x_n_stride: int = 0, y_n_stride: int = 0, res_n_stride: int = 0,
                 halo_mode: int = -1, w_batched: int = 0, w_ld: int = 0, w_h_stride: int = 0,
                 w_n_stride: int = 0, x_h_stride: int = 0, y_h_stride: int = 0, res_h_stride: int = 0,
                 y_tma_mode: int = -1, trace: Optional[torch.Tensor] = None, name: str = "conv_gemm",
                 peer_mode: int = 0, peer_rows: int = 0, peer_rank: int = 0, peer_world: int = 0,
                 peer_ptrs: Optional[Sequence[int]] = None, peer_counters: Optional[Sequence[int]] = None,
                 peer_ready: Optional[torch.Tensor] = None, peer_copiers: int = 0,
                 scale_a: Optional[torch.Tensor] = None, scale_b: Optional[torch.Tensor] = None,
                 pair_mode: int = -1, out_scale: float = 1.0):
        n, h, w_, cin = in_shape
        d = _ConvGemmDesc()
        self.status = status or StatusWord(x.device)
        d.x, d.w, d.y = x.data_ptr(), w_packed.data_ptr(), y.data_ptr()
        d.bias = bias.data_ptr() if bias is not None else None
        d.residual = residual.data_ptr() if residual is not None else None
        d.status = self.status.ptr
        d.dtype, d.out_dtype = dtype_code(x.dtype), dtype_code(y.dtype)
        d.N, d.H, d.W, d.Cin = n, h, w_, cin
        d.x_ld = x_ld if x_ld is not None else cin
        d.Ho, d.Wo, d.Cout = out_hw[0], out_hw[1], cout
        d.y_ld = y_ld if y_ld is not None else cout
        d.KH, d.KW, d.stride, d.pad_h, d.pad_w = kernel[0], kernel[1], stride, pad[0], pad[1]
        d.res_ld = res_ld if res_ld is not None else cout
        d.res_mode = res_mode if residual is not None else 0
        d.act, d.act_alpha, d.act_beta = ACT[act], act_alpha, act_beta
        d.tile_w, d.tile_h, d.block_n, d.max_ctas = tile[0], tile[1], block_n, max_ctas
        d.x_n_stride, d.y_n_stride, d.res_n_stride = x_n_stride, y_n_stride, res_n_stride
        d.halo_mode = halo_mode
        d.w_batched, d.w_ld, d.w_h_stride, d.w_n_stride = int(w_batched), w_ld, w_h_stride, w_n_stride
        d.x_h_stride, d.y_h_stride, d.res_h_stride = x_h_stride, y_h_stride, res_h_stride
        d.y_tma_mode = y_tma_mode
        d.trace = trace.data_ptr() if trace is not None else None
        self.trace = trace
        d.peer_mode, d.peer_rows, d.peer_rank, d.peer_world = peer_mode, peer_rows, peer_rank, peer_world
        for i, ptr in enumerate(peer_ptrs or []):
            d.peer_ptrs[i] = ptr
        for i, ptr in enumerate(peer_counters or []):
            d.peer_counters[i] = ptr
        d.peer_ready = peer_ready.data_ptr() if peer_ready is not None else None
        d.peer_copiers = peer_copiers
        self.peer_ready = peer_ready
        d.scale_a = scale_a.data_ptr() if scale_a is not None else None
        d.scale_b = scale_b.data_ptr() if scale_b is not None else None
        self.scales = (scale_a, scale_b)
        d.pair_mode = pair_mode
        d.out_scale = out_scale
        if bias is not None:
            assert bias.dtype == torch.float32
        if residual is not None:
            assert residual.dtype == x.dtype
        assert w_packed.dtype == x.dtype
        handle = _lib().fdb_conv_gemm_create(ctypes.byref(d))
        super().__init__(handle, [x, w_packed, y, bias, residual, self.status], name)
        self.create = ("fdb_conv_gemm_create", None, d)
        es_in, es_out = x.element_size(), y.element_size()
        # shape record for profilers: algorithmic FLOPs and bytes of this launch
        self.meta = dict(in_shape=(n, h, w_, cin), cin_logical=cin, out_hw=tuple(out_hw), cout=cout,
                         kernel=tuple(kernel), stride=stride,
                         bytes=n * h * w_ * cin * es_in + n * out_hw[0] * out_hw[1] * cout * es_out
                         + w_packed.numel() * es_in + (n * out_hw[0] * out_hw[1] * cout * es_in if residual is not None else 0))

    def info(self):
        out = (ctypes.c_int * 5)()
        _lib().fdb_conv_gemm_info(self.handle, out)
        return dict(tile_w=out[0], tile_h=out[1], block_n=out[2], grid=out[3], tiles=out[4],
                    variant=_lib().fdb_conv_gemm_variant(self.handle))


def conv2d_nhwc(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None, *, stride: int = 1,
                pad: int = 0, act: Optional[str] = None, residual: Optional[torch.Tensor] = None,
                res_mode: int = 0, out_dtype: Optional[torch.dtype] = None, **kw) -> torch.Tensor:
    """Eager convenience wrapper: ``x`` NHWC, ``weight`` ``[Cout,Cin,KH,KW]`` (any float dtype)."""
    n, h, w_, cin = x.shape
    cout, _, kh, kwid = weight.shape
    ho = (h + 2 * pad - kh) // stride + 1
    wo = (w_ + 2 * pad - kwid) // stride + 1
    wp = pack_conv_weight(weight, x.dtype)
    y = torch.empty(n, ho, wo, cout, dtype=out_dtype or x.dtype, device=x.device)
    b = bias.float().contiguous() if bias is not None else None
    op = ConvGemm(x, wp, y, in_shape=(n, h, w_, cin), out_hw=(ho, wo), cout=cout, kernel=(kh, kwid), stride=stride,
                  pad=(pad, pad), bias=b, residual=residual, res_mode=res_mode, act=act, **kw)
    op.launch()
    op.status.check("conv2d_nhwc")
    return y


def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None, *, act: Optional[str] = None,
           residual: Optional[torch.Tensor] = None, res_mode: int = 0, out_dtype: Optional[torch.dtype] = None,
           **kw) -> torch.Tensor:
    """Eager ``act(x @ weight.T + bias)`` for ``x [M,K]``, ``weight [N,K]``."""
    m, k = x.shape
    nout = weight.shape[0]
    wp = pack_linear_weight(weight, x.dtype)
    y = torch.empty(m, nout, dtype=out_dtype or x.dtype, device=x.device)
    b = bias.float().contiguous() if bias is not None else None
    op = ConvGemm(x, wp, y, in_shape=(1, 1, m, k), out_hw=(1, m), cout=nout, bias=b, residual=residual,
                  res_mode=res_mode, act=act, **kw)
    op.launch()
    op.status.check("linear")
    return y


# ------------------------------------------------------------------ fp8 (e4m3) operands
FP8_MAX = 448.0
K_BLOCK_FP8 = 128


def quantize_rows_e4m3(x: torch.Tensor):
    """Per-row symmetric quantisation to e4m3: returns ``(q [rows, K] float8_e4m3fn, scale [rows] fp32)`` with
    ``x ~= q * scale[:, None]``; the scale maps the row's absolute maximum onto 448."""
    xf = x.float()
    amax = xf.abs().amax(dim=1).clamp_min(1e-12)
    scale = amax / FP8_MAX
    q = (xf / scale[:, None]).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn)
    return q, scale.contiguous()


def pack_linear_weight_fp8(w: torch.Tensor):
    """``[N, K]`` weight -> (e4m3 ``[N, K padded to 128]``, per-output-channel scale ``[N]``)."""
    q, scale = quantize_rows_e4m3(w)
    n, k = q.shape
    kp = (k + K_BLOCK_FP8 - 1) // K_BLOCK_FP8 * K_BLOCK_FP8
    out = torch.zeros(n, kp, dtype=torch.float8_e4m3fn, device=w.device)
    out[:, :k] = q
    return out, scale


def linear_fp8(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None, act: Optional[str] = None,
               out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """``act(x @ w.T + bias)`` with both operands quantised to e4m3 on the fly (per token / per output channel
    scales) and multiplied by tcgen05 ``kind::f8f6f4`` MMAs with fp32 accumulation. This is per-channel-scaled fp8;
    the MX block-scaled form (one ue8m0 scale per 32 elements, scales in tensor memory) is not implemented."""
    m, k = x.shape
    n = w.shape[0]
    assert k % 16 == 0 and w.shape[1] == k
    xq, sa = quantize_rows_e4m3(x)
    wq, sb = pack_linear_weight_fp8(w)
    y = torch.empty(m, (n + 7) // 8 * 8, dtype=out_dtype, device=x.device)
    b = bias.float().contiguous() if bias is not None else None
    op = ConvGemm(xq, wq, y, in_shape=(1, 1, m, k), out_hw=(1, m), cout=n, bias=b, act=act, x_ld=k, y_ld=y.stride(0),
                  scale_a=sa, scale_b=sb, name="linear_fp8")
    op.launch()
    op.status.check("linear_fp8")
    return y[:, :n]
