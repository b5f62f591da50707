"""Single-kernel cases for timing and for profiler captures.

    python -m fastdeploy_b200.utils.kernel_cases conv --n 16 --hw 160 --cin 48 --cout 48 --k 3
    python -m fastdeploy_b200.utils.kernel_cases gemm --m 8192 --k 4096 --n 4096
    python -m fastdeploy_b200.utils.kernel_cases attention --b 64 --heads 16 --s 257 --d 80 --dtype bf16
    python -m fastdeploy_b200.utils.kernel_cases nms --n 8 --m 8400 --cout 80            (images, boxes, classes)
    python -m fastdeploy_b200.utils.kernel_cases preproc --n 8                           (1080x1920 frames -> 640x640)
    python -m fastdeploy_b200.utils.kernel_cases slot_reduce_ln --m 8192 --n 1280 --b 8  (rows, columns, ranks' partials)
    python -m fastdeploy_b200.utils.kernel_cases db_postprocess --n 2 --hw 960           (probability maps)

Each run launches the kernel ``--iters`` times after ``--warmup`` launches, times it with CUDA events
and prints one JSON line (time, TFLOP/s, bytes moved, and the fractions of ``--peak-tflops`` /
``--peak-gbs`` when those measured peaks of the GPU are given).
"""
from __future__ import annotations

import argparse
import json
import os
import sys


def main(argv=None) -> int:
    import torch
    from ..ops.conv_gemm import ConvGemm, pack_conv_weight, pack_linear_weight
    ap = argparse.ArgumentParser()
    ap.add_argument("kind", choices=["conv", "gemm", "attention", "nms", "preproc", "slot_reduce_ln", "db_postprocess", "layernorm"])
    ap.add_argument("--n", type=int, default=16)
    ap.add_argument("--hw", type=int, default=160)
    ap.add_argument("--cin", type=int, default=48)
    ap.add_argument("--cout", type=int, default=48)
    ap.add_argument("--k", type=int, default=3)
    ap.add_argument("--stride", type=int, default=1)
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--act", default="silu")
    ap.add_argument("--dtype", default="fp16")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--halo", type=int, default=-1)
    ap.add_argument("--block-n", type=int, default=0)
    ap.add_argument("--y-tma", type=int, default=-1)
    ap.add_argument("--pair", type=int, default=-1, help="CTA pairs (cta_group::2): -1 choose, 0 never, 1 force")
    ap.add_argument("--peak-tflops", type=float, default=0.0, help="measured dense 16-bit GEMM peak of this GPU")
    ap.add_argument("--peak-gbs", type=float, default=0.0, help="measured copy bandwidth of this GPU")
    ap.add_argument("--flush-l2", action="store_true", help="write 256 MB between timed launches")
    ap.add_argument("--b", type=int, default=64)
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--s", type=int, default=257)
    ap.add_argument("--d", type=int, default=80)
    ap.add_argument("--varlen", action="store_true", help="attention: packed sequences with lengths uniform in 16..s")
    a = ap.parse_args(argv)
    dt = torch.float16 if a.dtype == "fp16" else torch.bfloat16
    dev = "cuda"
    if a.kind in ("nms", "preproc", "slot_reduce_ln", "db_postprocess", "layernorm"):
        return _aux_case(a, dt)
    if a.kind == "conv":
        n, h, cin, cout, k, s = a.n, a.hw, a.cin, a.cout, a.k, a.stride
        p = k // 2
        ho = (h + 2 * p - k) // s + 1
        x = (torch.randn(n, h, h, cin, device=dev) * 0.5).to(dt)
        w = (torch.randn(cout, cin, k, k, device=dev) * 0.05).to(dt)
        b = torch.randn(cout, device=dev)
        y = torch.empty(n, ho, ho, cout, device=dev, dtype=dt)
        op = ConvGemm(x, pack_conv_weight(w, dt), y, in_shape=(n, h, h, cin), out_hw=(ho, ho), cout=cout,
                      kernel=(k, k), stride=s, pad=(p, p), bias=b, act=a.act if a.act != "none" else None,
                      halo_mode=a.halo, block_n=a.block_n, y_tma_mode=a.y_tma, pair_mode=a.pair)
        flops = 2.0 * n * ho * ho * cout * cin * k * k
        nbytes = x.numel() * 2 + y.numel() * 2 + w.numel() * 2
    elif a.kind == "attention" and a.varlen:
        # padding-free batch: b sequences back to back, the kernel reads starts and lengths from device memory
        from ..ops.transformer import PackedAttention, pack_offsets
        b, h, s, d = a.b, a.heads, a.s, a.d
        g = torch.Generator().manual_seed(0)
        lens = torch.randint(16, s + 1, (b,), generator=g).tolist()
        starts, rows = pack_offsets(lens)
        rows = (rows + 127) // 128 * 128
        qkv = (torch.randn(rows, 3 * h * d, device=dev) * 0.5).to(dt)
        o = torch.zeros(rows, h * d, device=dev, dtype=dt)
        att = PackedAttention(qkv[:, :h * d], qkv[:, h * d:2 * h * d], qkv[:, 2 * h * d:], o, heads=h, scale=d ** -0.5,
                              max_len=s, seq_start=torch.tensor(starts, dtype=torch.int32, device=dev),
                              seq_len=torch.tensor(lens, dtype=torch.int32, device=dev))
        att.ops[0].launch()
        op = att.ops[1]
        op.status = att.status
        op.info = lambda: {"kernel": "attention_sm100", "packed_rows": rows, "tokens": int(sum(lens))}
        flops = 4.0 * h * d * sum(n * n for n in lens)
        nbytes = (qkv.numel() + o.numel()) * 2
    elif a.kind == "attention":
        from ..ops.transformer import Attention
        b, h, s, d = a.b, a.heads, a.s, a.d
        qkv = (torch.randn(b, s, 3 * h * d, device=dev) * 0.5).to(dt)
        o = torch.zeros(b, s, h * d, device=dev, dtype=dt)
        att = Attention(qkv[..., :h * d], qkv[..., h * d:2 * h * d], qkv[..., 2 * h * d:], o, heads=h, scale=d ** -0.5,
                        fused=True)
        att.ops[0].launch()          # V^T once; the timed launch is the fused kernel alone
        op = att.ops[1]
        op.status = att.status
        op.info = lambda: {"kernel": "attention_sm100"}
        flops = 4.0 * b * h * s * s * d
        nbytes = (qkv.numel() + o.numel()) * 2
    else:
        m, kk, nn = a.m, a.k if a.k > 8 else 4096, a.n if a.n > 16 else 4096
        x = (torch.randn(m, kk, device=dev) * 0.5).to(dt)
        w = (torch.randn(nn, kk, device=dev) * 0.05).to(dt)
        y = torch.empty(m, nn, device=dev, dtype=dt)
        gemm_act = a.act if a.act not in ("none", "silu") or "--act" in (argv or sys.argv) else None
        op = ConvGemm(x, pack_linear_weight(w, dt), y, in_shape=(1, 1, m, kk), out_hw=(1, m), cout=nn,
                      bias=torch.randn(nn, device=dev) if gemm_act else None, act=gemm_act if gemm_act != "none" else None,
                      block_n=a.block_n, y_tma_mode=a.y_tma, pair_mode=a.pair)
        flops = 2.0 * m * kk * nn
        nbytes = (x.numel() + y.numel() + w.numel()) * 2
    for _ in range(a.warmup):
        op.launch()
    torch.cuda.synchronize()
    if a.flush_l2:
        flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
        times = []
        for _ in range(a.iters):
            flush.fill_(1)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            op.launch()
            e1.record()
            e1.synchronize()
            times.append(e0.elapsed_time(e1))
        times.sort()
        ms = times[len(times) // 2]
    else:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(a.iters):
            op.launch()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / a.iters
    op.status.check()
    out = {"case": vars(a), "ms": round(ms, 4), "tflops": round(flops / ms / 1e9, 1),
           "gbytes_per_s": round(nbytes / ms / 1e6, 1), "info": op.info()}
    if a.peak_tflops > 0:
        out["frac_of_measured_tflops_peak"] = round(out["tflops"] / a.peak_tflops, 3)
    if a.peak_gbs > 0:
        out["frac_of_measured_hbm"] = round(out["gbytes_per_s"] / a.peak_gbs, 3)
    print(json.dumps(out))
    return 0


class _Launch:
    """Adapter: a callable as the thing the timing loop launches."""

    def __init__(self, fn, status=None):
        self.fn, self.status = fn, status

    def launch(self):
        self.fn()


def _aux_case(a, dt) -> int:
    """Kernels outside the GEMM / attention family: one launch group each, timed like the others."""
    import numpy as np
    import torch
    dev = "cuda"
    g = torch.Generator(device="cpu").manual_seed(0)
    info = {}
    if a.kind == "nms":
        from ..ops.nms import MulticlassNMS
        n, m, c = a.n, a.m if a.m != 8192 else 8400, a.cout if a.cout != 48 else 80
        centre = torch.rand(n, m, 2, generator=g) * 600
        size = torch.rand(n, m, 2, generator=g) * 80 + 8
        boxes = torch.cat([centre - size / 2, centre + size / 2], -1).to(dev)
        scores = (torch.rand(n, m, c, generator=g) ** 6).to(dev).half()             # anchor-major fp16, as the head writes them
        nms = MulticlassNMS(boxes, scores, class_major=False, score_threshold=0.01, nms_threshold=0.6, nms_top_k=1000,
                            keep_top_k=100)
        op = _Launch(nms.launch)
        nbytes = boxes.numel() * 4 + scores.numel() * 2
        info = {"kernel": "multiclass_nms", "launches": nms.launches, "images": n, "boxes": m, "classes": c}
    elif a.kind == "preproc":
        from ..ops import preproc as P
        n, h, w = a.n, 1080, 1920
        raw = torch.randint(0, 256, (n, h, w, 3), generator=g, dtype=torch.uint8).to(dev)
        meta_host = np.zeros(n, dtype=P.IMAGE_META)
        for i in range(n):
            P.fill_meta(meta_host, i, src_offset=i * h * w * 3, src_hw=(h, w), src_stride=w * 3, resized_hw=(640, 640))
        meta = torch.from_numpy(meta_host.view(np.uint8).copy()).to(dev)
        dst = torch.zeros(n, 640, 640, 8, dtype=dt, device=dev)
        alpha, beta = P.normalize_coeffs([0.485, 0.456, 0.406], [0.229, 0.224, 0.225])
        pre = P.Preprocess(raw.view(-1), meta, dst, n=n, out_hw=(640, 640), layout="nhwc", c_out=8, interp="linear",
                           swap_rb=True, alpha=alpha, beta=beta)
        op = _Launch(pre.launch)
        nbytes = raw.numel() + dst.numel() * 2
        info = {"kernel": "preproc", "frames": n, "src": [h, w], "dst": [640, 640]}
    elif a.kind == "layernorm":
        from ..ops import transformer as T
        from ..ops.base import StatusWord
        rows, cols = a.m, a.n if a.n != 16 else 768
        x = (torch.randn(rows, cols, generator=g) * 0.5).to(dev).to(dt)
        y = torch.zeros(rows, cols, device=dev, dtype=dt)
        gamma, beta = (torch.rand(cols, generator=g) + 0.5).to(dev), torch.randn(cols, generator=g).to(dev)
        ln = T.layernorm(x, y, gamma, beta, rows=rows, c=cols, eps=1e-5, x_ld=cols, y_ld=cols)
        op = _Launch(ln.launch, StatusWord(torch.device(dev)))
        nbytes = 2 * x.numel() * 2
        info = {"kernel": "layernorm", "rows": rows, "cols": cols}
    elif a.kind == "slot_reduce_ln":
        import ctypes
        from ..ops.base import StatusWord, current_stream_ptr, dtype_code
        from ..parallel.comm import _lib
        rows, cols, world = a.m, a.n if a.n != 16 else 1280, a.b if a.b != 64 else 8
        slots = (torch.randn(world, rows, cols, generator=g) * 0.3).to(dev).bfloat16()
        x0 = torch.randn(rows, cols, generator=g).to(dev).bfloat16()
        x = x0.clone()
        bias = torch.randn(cols, generator=g).to(dev)
        gamma, beta = (torch.rand(cols, generator=g) + 0.5).to(dev), torch.randn(cols, generator=g).to(dev)
        y = torch.zeros(rows, cols, device=dev, dtype=torch.bfloat16)
        counters = torch.full(((rows + 127) // 128,), 7, dtype=torch.int32, device=dev)    # arrivals already complete
        st = StatusWord(torch.device(dev))
        Pv = ctypes.c_void_p

        def launch():
            rc = _lib().fdb_comm_slot_reduce_ln(Pv(slots.data_ptr()), Pv(counters.data_ptr()), 7, Pv(x.data_ptr()),
                                                Pv(bias.data_ptr()), rows, cols, world, dtype_code(torch.bfloat16), st.ptr,
                                                Pv(gamma.data_ptr()), Pv(beta.data_ptr()), 1e-6, Pv(y.data_ptr()), cols,
                                                Pv(current_stream_ptr()), 0, 1.0)
            if rc != 0:
                raise RuntimeError("slot_reduce_ln failed")
        op = _Launch(launch, st)
        nbytes = slots.numel() * 2 + 3 * x.numel() * 2           # partials and the residual in, residual and LayerNorm out
        info = {"kernel": "slot_reduce_ln", "rows": rows, "cols": cols, "partials": world}
    else:
        from ..ops.postproc import DBPostprocess
        n, hw = a.n, a.hw if a.hw != 160 else 960
        prob = torch.rand(n, hw, hw, generator=g) * 0.1
        for i in range(n):
            for _ in range(45):                                     # text-line rectangles
                hh, ww = int(torch.randint(16, 40, (1,), generator=g)), int(torch.randint(60, 400, (1,), generator=g))
                y0 = int(torch.randint(0, hw - hh, (1,), generator=g))
                x0p = int(torch.randint(0, hw - ww, (1,), generator=g))
                prob[i, y0:y0 + hh, x0p:x0p + ww] = 0.9
        buf = torch.zeros(n, hw, hw, 8, dtype=dt, device=dev)
        buf[..., 0] = prob.to(dev).to(dt)
        db = DBPostprocess(n, hw, hw, dev)
        db.set_info([(hw, hw, hw, hw)] * n)
        view = buf[..., 0]
        op = _Launch(lambda: db.run(view))
        nbytes = n * hw * hw * (2 + 4 * 6)
        info = {"kernel": "db_postprocess", "launches": db.launches, "maps": n, "size": hw}
    for _ in range(a.warmup):
        op.launch()
    torch.cuda.synchronize()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev) if a.flush_l2 else None
    times = []
    for _ in range(a.iters):
        if flush is not None:
            flush.fill_(1)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        op.launch()
        e1.record()
        e1.synchronize()
        times.append(e0.elapsed_time(e1))
    times.sort()
    ms = times[len(times) // 2]
    if op.status is not None:
        op.status.check()
    if a.kind == "db_postprocess":
        info["boxes_found"] = [len(b) for b in db.boxes()[0]]
    out = {"case": vars(a), "ms": round(ms, 4), "gbytes_per_s": round(nbytes / ms / 1e6, 1), "info": info}
    if a.peak_gbs > 0:
        out["frac_of_measured_hbm"] = round(out["gbytes_per_s"] / a.peak_gbs, 3)
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
