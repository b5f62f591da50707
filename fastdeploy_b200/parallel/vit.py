"""Tensor-parallel Vision Transformer (ViT-H/14 and smaller) over the fused GEMM + collective kernels.

Activations between blocks are *row sharded*: the ``B * T`` token rows (padded to ``world * 128 * j``)
are split evenly over the ranks, and the residual stream, both LayerNorms and the residual additions
only ever touch a rank's own rows. Each encoder block is four tensor-core launches with their
collectives inside:

  LayerNorm -> [all-gather -> QKV GEMM]     column parallel, this rank's heads only
  attention over the local heads            one fused tcgen05 kernel (scores stay in tensor memory)
  [proj GEMM -> reduce-scatter] + residual + LayerNorm   row parallel, partial sums land in the owner's
                                            slots; one kernel sums them, adds the residual and normalises
  [all-gather -> fc1 GEMM + GELU]
  [fc2 GEMM -> reduce-scatter] + residual + the next block's LayerNorm

Buffers are shared by all layers. The two all-gather inputs alternate between two heap buffers, so
the one device barrier in front of each all-gather GEMM is also what keeps a fast rank from
overwriting a shard that a slow rank is still pulling (a rank can only write buffer A again after
the barrier in front of the GEMM that reads buffer B, which every rank reaches after its own read of
A). The two reduce-scatters alternate between two slot buffers with monotonic arrival counters.

The reference serves ViT through ``PaddleClasModel`` on one GPU
(fastdeploy/vision/classification/ppcls/model.cc:23-119); it has no tensor parallelism.
"""
from __future__ import annotations

import ctypes
import math
from typing import Callable, Dict, Optional

import torch

from .. import _native
from ..ops.base import current_stream_ptr, dtype_code
from ..ops.conv_gemm import ConvGemm, pack_linear_weight, pack_linear_weight_fp8
from ..ops.nhwc import quantize_e4m3
from ..ops.transformer import Attention, layernorm
from .comm import Communicator, _lib

VIT_SIZES = {
    "huge14": dict(patch=14, layers=32, hidden=1280, heads=16, mlp=5120),
    "large16": dict(patch=16, layers=24, hidden=1024, heads=16, mlp=4096),
    "base16": dict(patch=16, layers=12, hidden=768, heads=12, mlp=3072),
    "test": dict(patch=14, layers=2, hidden=128, heads=4, mlp=256),
    "test8": dict(patch=14, layers=2, hidden=256, heads=8, mlp=512),     # divisible over 8 ranks
}


def random_vit_weights(cfg: Dict[str, int], image: int, num_classes: int, seed: int = 0,
                       device: str = "cpu") -> Dict[str, torch.Tensor]:
    """Seeded random weights in torch layout (``[out, in]`` linears). Every rank calling this with the
    same seed gets the same tensors."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    H, F, P = cfg["hidden"], cfg["mlp"], cfg["patch"]
    T = (image // P) ** 2 + 1

    def rn(*shape, s=0.02):
        return (torch.randn(*shape, generator=g) * s).to(device)

    w = {"patch_w": rn(H, 3, P, P), "patch_b": rn(H), "cls": rn(H), "pos": rn(T, H),
         "norm_g": 1.0 + rn(H, s=0.05), "norm_b": rn(H), "head_w": rn(num_classes, H), "head_b": rn(num_classes)}
    for l in range(cfg["layers"]):
        p = f"blocks.{l}."
        w[p + "ln1_g"], w[p + "ln1_b"] = 1.0 + rn(H, s=0.05), rn(H)
        w[p + "ln2_g"], w[p + "ln2_b"] = 1.0 + rn(H, s=0.05), rn(H)
        for nm in ("q", "k", "v", "proj"):
            w[p + nm + "_w"], w[p + nm + "_b"] = rn(H, H), rn(H)
        w[p + "fc1_w"], w[p + "fc1_b"] = rn(F, H), rn(F)
        w[p + "fc2_w"], w[p + "fc2_b"] = rn(H, F), rn(H)
    return w


def vit_reference(w: Dict[str, torch.Tensor], cfg: Dict[str, int], x: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """Plain fp32 PyTorch forward of the same network (the numerics oracle): ``x [B, 3, S, S]`` ->
    class probabilities ``[B, classes]``."""
    import torch.nn.functional as Fn
    H, NH, P = cfg["hidden"], cfg["heads"], cfg["patch"]
    D = H // NH
    B = x.shape[0]
    f = {k: v.float().to(x.device) for k, v in w.items()}
    y = Fn.conv2d(x.float(), f["patch_w"], f["patch_b"], stride=P).flatten(2).transpose(1, 2)
    y = torch.cat([f["cls"].view(1, 1, H).expand(B, 1, H), y], 1) + f["pos"][None]
    T = y.shape[1]
    for l in range(cfg["layers"]):
        p = f"blocks.{l}."
        h = Fn.layer_norm(y, (H,), f[p + "ln1_g"], f[p + "ln1_b"], eps)
        q, k, v = (Fn.linear(h, f[p + n + "_w"], f[p + n + "_b"]).view(B, T, NH, D).transpose(1, 2) for n in "qkv")
        a = torch.softmax(q @ k.transpose(-1, -2) * D ** -0.5, -1) @ v
        y = y + Fn.linear(a.transpose(1, 2).reshape(B, T, H), f[p + "proj_w"], f[p + "proj_b"])
        h = Fn.layer_norm(y, (H,), f[p + "ln2_g"], f[p + "ln2_b"], eps)
        y = y + Fn.linear(Fn.gelu(Fn.linear(h, f[p + "fc1_w"], f[p + "fc1_b"])), f[p + "fc2_w"], f[p + "fc2_b"])
    y = Fn.layer_norm(y, (H,), f["norm_g"], f["norm_b"], eps)
    return torch.softmax(Fn.linear(y[:, 0], f["head_w"], f["head_b"]), -1)


class TensorParallelViT:
    """ViT classifier over ``comm.world`` GPUs. ``forward(images)`` takes the full ``[B, 3, S, S]`` batch on
    every rank (fp16/bf16/fp32, on the device) and returns the ``[B, classes]`` probabilities on every rank."""

    def __init__(self, comm: Communicator, weights: Dict[str, torch.Tensor], cfg: Dict[str, int], *, batch: int,
                 image: int = 224, dtype: torch.dtype = torch.bfloat16, eps: float = 1e-6, name: str = "tpvit",
                 copiers: int = 0, precision: str = "", act_scales: Optional[Dict[str, float]] = None):
        """``precision="fp8"``: the four linears of every block run on e4m3 operands (``tcgen05.mma.kind::f8f6f4``,
        fp32 accumulation). Weights are quantised per output channel; activations with one static scale per
        tensor and layer (``act_scales``, from :meth:`calibrate` of a 16-bit instance or from a quantised model
        file): the LayerNorms and the fc1 epilogue write e4m3 directly, the attention output passes through one
        quantise kernel, so the gathered activations cross NVLink as bytes. The residual stream, attention and
        the partial sums of the row-parallel GEMMs stay in ``dtype``."""
        self.comm, self.cfg, self.dtype, self.eps = comm, cfg, dtype, eps
        self.fp8 = precision == "fp8"
        if self.fp8 and act_scales is None:
            raise ValueError("precision='fp8' needs act_scales (see TensorParallelViT.calibrate)")
        self.act_scales = act_scales or {}
        self.calib: Optional[Dict[str, float]] = None
        ws, r, dev = comm.world, comm.rank, comm.device
        H, NH, F, P, L = cfg["hidden"], cfg["heads"], cfg["mlp"], cfg["patch"], cfg["layers"]
        assert NH % ws == 0 and F % ws == 0 and H % 8 == 0
        D = H // NH
        hl, fl = NH // ws, F // ws
        hd = hl * D
        G = image // P
        T = G * G + 1
        self.B, self.T, self.H, self.G, self.P = batch, T, H, G, P
        m_real = batch * T
        unit = ws * 128
        self.M = M = (m_real + unit - 1) // unit * unit
        self.rows = rows = M // ws
        self.m_real = m_real
        es = 2

        def dv(t):
            return t.to(dev)

        # ---- patch embedding (replicated weights; each rank embeds the images its rows touch)
        self.row0 = r * rows
        self.row1 = min((r + 1) * rows, m_real)
        self.img0 = min(self.row0 // T, batch)
        self.img1 = min((max(self.row1, self.row0 + 1) - 1) // T + 1, batch) if self.row1 > self.row0 else self.img0
        kp = 3 * P * P
        self.kp_pad = (kp + 7) // 8 * 8
        nimg = max(self.img1 - self.img0, 1)
        self.patches = torch.zeros(nimg * G * G, self.kp_pad, dtype=dtype, device=dev)
        self.patch_w = pack_linear_weight(torch.nn.functional.pad(dv(weights["patch_w"]).reshape(H, kp),
                                                                  (0, self.kp_pad - kp)), dtype)
        self.patch_out = torch.empty(nimg * G * G, H, dtype=dtype, device=dev)
        self.patch_bias = dv(weights["patch_b"]).float().contiguous()
        self.patch_op = ConvGemm(self.patches, self.patch_w, self.patch_out, in_shape=(1, 1, nimg * G * G, self.kp_pad),
                                 out_hw=(1, nimg * G * G), cout=H, bias=self.patch_bias, status=comm.status,
                                 name=name + ".patch")
        self.cls_pos0 = (dv(weights["cls"]).float() + dv(weights["pos"])[0].float()).to(dtype)
        self.pos_rest = dv(weights["pos"])[1:].to(dtype)
        self.tokens = torch.zeros(nimg, T, H, dtype=dtype, device=dev)

        # ---- shared activation buffers
        self.xres = torch.zeros(rows, H, dtype=dtype, device=dev)            # residual stream, this rank's rows
        gdt = torch.float8_e4m3fn if self.fp8 else dtype          # what the all-gather GEMMs read
        self.gather_blocks = [comm.alloc(f"{name}.gather{i}", M * H * es) for i in range(2)]
        self.gathered = [comm.tensor(b, (M, H), gdt) for b in self.gather_blocks]
        self.shard = [g[r * rows:(r + 1) * rows] for g in self.gathered]
        self.qkv = torch.zeros(M, 3 * hd, dtype=dtype, device=dev)
        self.ctx = torch.zeros(M, hd, dtype=dtype, device=dev)
        self.ffn = torch.zeros(M, fl, dtype=gdt, device=dev)
        self.ctx_q = torch.zeros(M, hd, dtype=gdt, device=dev) if self.fp8 else None
        slot_bytes = ws * rows * H * es
        self.blocks128 = rows // 128
        cnt_bytes = (self.blocks128 * 4 + 1023) // 1024 * 1024
        self.slot_blocks = [comm.alloc(f"{name}.slots{i}", slot_bytes) for i in range(2)]
        self.cnt_blocks = [comm.alloc(f"{name}.cnt{i}", cnt_bytes) for i in range(2)]
        self.slots = [comm.tensor(b, (ws, rows, H), dtype) for b in self.slot_blocks]
        self.counters = [comm.tensor(b, (self.blocks128,), torch.int32) for b in self.cnt_blocks]
        self.targets = [0, 0]
        # this rank's rows inside every rank's partial-result buffer (the pull form of the reduce-scatter)
        row_off = r * rows * H * es
        self.part_ptrs = [(ctypes.c_void_p * 8)(*[comm.ptr(k, b) + row_off for k in range(ws)]) for b in self.slot_blocks]

        q3 = self.qkv[:m_real].view(batch, T, 3 * hd)
        self.attn = Attention(q3[:, :, 0:hd], q3[:, :, hd:2 * hd], q3[:, :, 2 * hd:3 * hd],
                              self.ctx[:m_real].view(batch, T, hd), heads=hl, scale=float(D) ** -0.5,
                              status=comm.status)

        # ---- per-layer ops
        self.fuse_ln = H <= 2048 and ws in (1, 2, 4, 8)     # slot reduction + residual + LayerNorm in one kernel
        self.layers = []
        gptr = [[comm.ptr(k, b) for k in range(ws)] for b in self.gather_blocks]
        sptr = [[comm.ptr(k, b) for k in range(ws)] for b in self.slot_blocks]
        cptr = [[comm.ptr(k, b) for k in range(ws)] for b in self.cnt_blocks]
        for l in range(L):
            p = f"blocks.{l}."
            lw = {k[len(p):]: v for k, v in weights.items() if k.startswith(p)}
            sl = slice(r * hd, (r + 1) * hd)
            w_qkv = torch.cat([dv(lw["q_w"][sl]), dv(lw["k_w"][sl]), dv(lw["v_w"][sl])])
            b_qkv = torch.cat([dv(lw["q_b"][sl]), dv(lw["k_b"][sl]), dv(lw["v_b"][sl])]).float().contiguous()
            lay = {}
            lay["ln1_gb"] = (dv(lw["ln1_g"]).float().contiguous(), dv(lw["ln1_b"]).float().contiguous())
            lay["ln2_gb"] = (dv(lw["ln2_g"]).float().contiguous(), dv(lw["ln2_b"]).float().contiguous())
            fs = slice(r * fl, (r + 1) * fl)
            if self.fp8:
                sc = self.act_scales
                s_h1, s_ctx, s_h2, s_ffn = sc[f"h1.{l}"], sc[f"ctx.{l}"], sc[f"h2.{l}"], sc[f"ffn.{l}"]
                lay["scales"] = (s_h1, s_ctx, s_h2, s_ffn)
                lay["ln1"] = layernorm(self.xres, self.shard[0], dv(lw["ln1_g"]).float(), dv(lw["ln1_b"]).float(),
                                       rows=rows, c=H, eps=eps, out_scale=1.0 / s_h1)
                lay["ln2"] = layernorm(self.xres, self.shard[1], dv(lw["ln2_g"]).float(), dv(lw["ln2_b"]).float(),
                                       rows=rows, c=H, eps=eps, out_scale=1.0 / s_h2)
                wq, sw = pack_linear_weight_fp8(w_qkv)
                lay["qkv"] = self._col(0, gptr[0], wq, b_qkv, self.qkv, 3 * hd, None, f"{name}.{l}.qkv", copiers,
                                       scale_b=(sw * s_h1).contiguous())
                wq, sw = pack_linear_weight_fp8(dv(lw["fc1_w"][fs]))
                lay["fc1"] = self._col(1, gptr[1], wq, dv(lw["fc1_b"][fs]).float().contiguous(), self.ffn, fl, "gelu",
                                       f"{name}.{l}.fc1", copiers, scale_b=(sw * s_h2).contiguous(), out_scale=1.0 / s_ffn)
                lay["ctx_q"] = quantize_e4m3(self.ctx, self.ctx_q, rows=M, c=hd, scale=1.0 / s_ctx)
                wq, sw = pack_linear_weight_fp8(dv(lw["proj_w"][:, sl]))
                lay["proj"] = self._row(0, sptr[0], cptr[0], self.ctx_q, hd, wq, f"{name}.{l}.proj",
                                        scale_b=(sw * s_ctx).contiguous())
                wq, sw = pack_linear_weight_fp8(dv(lw["fc2_w"][:, fs]))
                lay["fc2"] = self._row(1, sptr[1], cptr[1], self.ffn, fl, wq, f"{name}.{l}.fc2",
                                       scale_b=(sw * s_ffn).contiguous())
            else:
                lay["ln1"] = layernorm(self.xres, self.shard[0], dv(lw["ln1_g"]).float(), dv(lw["ln1_b"]).float(),
                                       rows=rows, c=H, eps=eps)
                lay["ln2"] = layernorm(self.xres, self.shard[1], dv(lw["ln2_g"]).float(), dv(lw["ln2_b"]).float(),
                                       rows=rows, c=H, eps=eps)
                lay["qkv"] = self._col(0, gptr[0], pack_linear_weight(w_qkv, dtype), b_qkv, self.qkv, 3 * hd, None,
                                       f"{name}.{l}.qkv", copiers)
                lay["fc1"] = self._col(1, gptr[1], pack_linear_weight(dv(lw["fc1_w"][fs]), dtype),
                                       dv(lw["fc1_b"][fs]).float().contiguous(), self.ffn, fl, "gelu", f"{name}.{l}.fc1",
                                       copiers)
                lay["proj"] = self._row(0, sptr[0], cptr[0], self.ctx, hd,
                                        pack_linear_weight(dv(lw["proj_w"][:, sl]), dtype), f"{name}.{l}.proj")
                lay["fc2"] = self._row(1, sptr[1], cptr[1], self.ffn, fl,
                                       pack_linear_weight(dv(lw["fc2_w"][:, fs]), dtype), f"{name}.{l}.fc2")
            lay["proj_b"] = dv(lw["proj_b"]).float().contiguous()
            lay["fc2_b"] = dv(lw["fc2_b"]).float().contiguous()
            self.layers.append(lay)

        # ---- head: final LayerNorm on the local rows, class rows summed over the ranks, replicated linear
        self.final = torch.zeros(rows, H, dtype=dtype, device=dev)
        self.ln_f_gb = (dv(weights["norm_g"]).float().contiguous(), dv(weights["norm_b"]).float().contiguous())
        self.ln_f = layernorm(self.xres, self.final, self.ln_f_gb[0], self.ln_f_gb[1], rows=rows, c=H, eps=eps)
        cls_rows = torch.arange(batch, device=dev) * T
        mine = (cls_rows >= self.row0) & (cls_rows < self.row0 + rows)
        self.cls_img = torch.nonzero(mine).flatten()
        self.cls_local = cls_rows[mine] - self.row0
        self.cls_feat = torch.zeros(batch, H, dtype=torch.float32, device=dev)
        self.head_w = dv(weights["head_w"]).float()
        self.head_b = dv(weights["head_b"]).float()

    # ------------------------------------------------------------------ op builders
    def _col(self, which, ptrs, w, bias, y, n_local, act, name, copiers, scale_b=None, out_scale=1.0):
        c = self.comm
        if c.world == 1:      # nothing to gather: a plain GEMM on the local buffer
            return ConvGemm(self.gathered[which], w, y, in_shape=(1, 1, self.M, self.H), out_hw=(1, self.M),
                            cout=n_local, bias=bias, act=act, x_ld=self.H, y_ld=y.stride(0), status=c.status, name=name,
                            scale_b=scale_b, out_scale=out_scale)
        ready = torch.zeros(self.M // 128, dtype=torch.int32, device=self.comm.device)
        return ConvGemm(self.gathered[which], w, y, in_shape=(1, 1, self.M, self.H), out_hw=(1, self.M), cout=n_local,
                        bias=bias, act=act, x_ld=self.H, y_ld=y.stride(0), status=c.status, name=name, peer_mode=1,
                        peer_rows=self.rows, peer_rank=c.rank, peer_world=c.world, peer_ptrs=ptrs, peer_ready=ready,
                        peer_copiers=copiers, scale_b=scale_b, out_scale=out_scale)

    def _row(self, which, slot_ptrs, cnt_ptrs, x, k_local, w, name, scale_b=None):
        c = self.comm
        if c.world == 1:      # the only slot is local: a plain GEMM writes it, stream order replaces the counters
            op = ConvGemm(x, w, self.slots[which].view(self.rows, self.H), in_shape=(1, 1, self.M, k_local),
                          out_hw=(1, self.M), cout=self.H, x_ld=x.stride(0), y_ld=self.H, status=c.status, name=name,
                          scale_b=scale_b)
            op.stores_per_block = 0
            return op
        # reduce-scatter by pulling: the partial [M, H] result stays in this rank's heap block (same layout as the
        # slot buffer: row block o belongs to rank o); the epilogue only bumps the owner's arrival counters, and
        # each rank's reduction kernel reads its rows from every peer over NVLink
        op = ConvGemm(x, w, self.slots[which].view(c.world * self.rows, self.H), in_shape=(1, 1, self.M, k_local),
                      out_hw=(1, self.M), cout=self.H, x_ld=x.stride(0), y_ld=self.H, status=c.status, name=name,
                      peer_mode=3 if self.fuse_ln else 2, peer_rows=self.rows, peer_rank=c.rank, peer_world=c.world,
                      peer_ptrs=slot_ptrs,
                      peer_counters=cnt_ptrs, scale_b=scale_b)
        info = op.info()
        bn = info["block_n"]
        n_tiles = (self.H + bn - 1) // bn
        op.stores_per_block = sum((min(self.H, (t + 1) * bn) - t * bn + 31) // 32 for t in range(n_tiles))
        return op

    def _reduce_into_residual(self, which: int, op, bias: torch.Tensor, ln=None) -> None:
        """Waits (bounded, per 128-row block) for every rank's partial block, then
        ``xres = xres + bias + sum of the partials``; with ``ln = (gamma, beta, out)`` the same kernel also writes
        ``out = LayerNorm(xres)``, i.e. the input of the next all-gather GEMM."""
        c = self.comm
        self.targets[which] += c.world * op.stores_per_block
        P = ctypes.c_void_p
        if ln is not None and c.world > 1:
            gamma, beta, out = ln[:3]
            out_scale = ln[3] if len(ln) > 3 else 1.0
            out8 = out.dtype == torch.float8_e4m3fn
            rc = _lib().fdb_comm_slot_reduce_ln_pull(
                self.part_ptrs[which], P(self.counters[which].data_ptr()), self.targets[which],
                P(self.xres.data_ptr()), P(bias.data_ptr()), self.rows, self.H, c.world, dtype_code(self.dtype),
                c.status.ptr, P(gamma.data_ptr()), P(beta.data_ptr()), self.eps, P(out.data_ptr()), out.stride(0),
                P(current_stream_ptr()), int(out8), float(out_scale))
        elif ln is not None:
            gamma, beta, out = ln[:3]
            out_scale = ln[3] if len(ln) > 3 else 1.0
            out8 = out.dtype == torch.float8_e4m3fn
            rc = _lib().fdb_comm_slot_reduce_ln(
                P(self.slots[which].data_ptr()), P(self.counters[which].data_ptr()), self.targets[which],
                P(self.xres.data_ptr()), P(bias.data_ptr()), self.rows, self.H, c.world, dtype_code(self.dtype),
                c.status.ptr, P(gamma.data_ptr()), P(beta.data_ptr()), self.eps, P(out.data_ptr()), out.stride(0),
                P(current_stream_ptr()), int(out8), float(out_scale))
        else:
            rc = _lib().fdb_comm_slot_reduce_res(
                P(self.slots[which].data_ptr()), P(self.counters[which].data_ptr()), self.targets[which],
                P(self.xres.data_ptr()), P(bias.data_ptr()), P(self.xres.data_ptr()), self.H, self.rows, self.H, self.H,
                self.H, c.world, dtype_code(self.dtype), c.status.ptr, P(current_stream_ptr()))
        if rc != 0:
            raise RuntimeError("tp vit: " + _native.last_error())

    # ------------------------------------------------------------------ forward
    def embed(self, images: torch.Tensor) -> None:
        """Patch embedding + class token + position embedding for this rank's rows -> ``xres``."""
        B, T, H, G, P = self.B, self.T, self.H, self.G, self.P
        n = self.img1 - self.img0
        self.xres.zero_()
        if n <= 0:
            return
        x = images[self.img0:self.img1].to(self.dtype)
        pt = x.view(n, 3, G, P, G, P).permute(0, 2, 4, 1, 3, 5).reshape(n * G * G, 3 * P * P)
        self.patches[:, :3 * P * P].copy_(pt)
        self.patch_op.launch()
        self.tokens[:n, 0] = self.cls_pos0
        torch.add(self.patch_out.view(-1, G * G, H)[:n], self.pos_rest[None], out=self.tokens[:n, 1:])
        flat = self.tokens[:n].view(n * T, H)
        lo = self.row0 - self.img0 * T
        cnt = self.row1 - self.row0
        self.xres[:cnt].copy_(flat[lo:lo + cnt])

    def encoder(self) -> None:
        """All encoder blocks and the final LayerNorm: ``xres`` -> ``final``. Every LayerNorm except the first
        rides on the slot reduction in front of it (``fuse_ln``)."""
        c = self.comm
        n = len(self.layers)
        real = max(self.row1 - self.row0, 0)          # this rank's rows that carry tokens (the rest is padding)
        rec = self._record if self.calib is not None else (lambda *a: None)
        for l, lay in enumerate(self.layers):
            if l == 0 or not self.fuse_ln:
                lay["ln1"].launch()
            rec(f"h1.{l}", self.shard[0][:real])
            c.barrier()
            lay["qkv"].launch()
            self.attn.launch()
            rec(f"ctx.{l}", self.ctx[:self.m_real])
            if self.fp8:
                lay["ctx_q"].launch()
            lay["proj"].launch()
            if self.fuse_ln:
                ln2 = lay["ln2_gb"] + (self.shard[1],) + ((1.0 / lay["scales"][2],) if self.fp8 else ())
                self._reduce_into_residual(0, lay["proj"], lay["proj_b"], ln2)
            else:
                self._reduce_into_residual(0, lay["proj"], lay["proj_b"])
                lay["ln2"].launch()
            rec(f"h2.{l}", self.shard[1][:real])
            c.barrier()
            lay["fc1"].launch()
            rec(f"ffn.{l}", self.ffn[:self.m_real])
            lay["fc2"].launch()
            if self.fuse_ln:
                if l + 1 < n:
                    nxt = self.layers[l + 1]["ln1_gb"] + (self.shard[0],) + \
                        ((1.0 / self.layers[l + 1]["scales"][0],) if self.fp8 else ())
                else:
                    nxt = self.ln_f_gb + (self.final,)
                self._reduce_into_residual(1, lay["fc2"], lay["fc2_b"], nxt)
            else:
                self._reduce_into_residual(1, lay["fc2"], lay["fc2_b"])
        if not self.fuse_ln:
            self.ln_f.launch()

    # ------------------------------------------------------------------ fp8 calibration
    def _record(self, key: str, t: torch.Tensor) -> None:
        v = float(t.float().abs().max()) if t.numel() else 0.0
        self.calib[key] = max(self.calib.get(key, 0.0), v)

    def calibrate(self, images: torch.Tensor, margin: float = 1.0) -> Dict[str, float]:
        """Runs one forward of this (16-bit) model on sample ``images`` and returns the static activation scales
        of the fp8 form: per layer the absolute maximum of the four GEMM inputs (both LayerNorm outputs, the
        attention output, the GELU output), maximum over the ranks, divided by the e4m3 range 448 (times
        ``margin``). This is the post-training-quantisation recipe of the reference's int8 path (static
        per-tensor activation scales from calibration data) with fp8 as the storage type."""
        assert not self.fp8, "calibrate a 16-bit instance"
        self.calib = {}
        try:
            self.forward(images)
            torch.cuda.synchronize()
            keys = sorted(self.calib)
            t = torch.tensor([self.calib[k] for k in keys], device=self.comm.device, dtype=torch.float32)
            if self.comm.world > 1:
                self.comm.dist.all_reduce(t, op=self.comm.dist.ReduceOp.MAX, group=self.comm.group)
            return {k: max(float(v), 1e-6) * margin / 448.0 for k, v in zip(keys, t.tolist())}
        finally:
            self.calib = None

    def head(self) -> torch.Tensor:
        self.cls_feat.zero_()
        if self.cls_img.numel():
            self.cls_feat[self.cls_img] = self.final[self.cls_local].float()
        if self.comm.world > 1:
            self.comm.dist.all_reduce(self.cls_feat, group=self.comm.group)
        return torch.softmax(torch.addmm(self.head_b, self.cls_feat, self.head_w.t()), -1)

    def forward(self, images: torch.Tensor) -> torch.Tensor:
        self.embed(images)
        self.encoder()
        return self.head()

    @property
    def launches_per_forward(self) -> int:
        """Native kernel launches per forward: per layer 2 barriers, 4 GEMMs, 2 attention launches and 2 slot
        reductions (with the LayerNorms inside), plus the patch GEMM and the first LayerNorm."""
        per_layer = 2 + 4 + len(self.attn.ops) + 2 + (0 if self.fuse_ln else 2) + (1 if self.fp8 else 0)
        return len(self.layers) * per_layer + 2

    def flops(self) -> float:
        H, F, T, B, L = self.H, self.cfg["mlp"], self.T, self.B, len(self.layers)
        per_tok = 2.0 * (4 * H * H + 2 * H * F)
        attn = 4.0 * T * T * H
        return L * B * (T * per_tok + attn)
