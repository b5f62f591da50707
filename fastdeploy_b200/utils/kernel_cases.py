"""Single-kernel cases for timing and for profiler captures.

    python -m fastdeploy_b200.utils.kernel_cases conv --n 16 --hw 160 --cin 48 --cout 48 --k 3
    python -m fastdeploy_b200.utils.kernel_cases gemm --m 8192 --k 4096 --n 4096
    python -m fastdeploy_b200.utils.kernel_cases attention --b 64 --heads 16 --s 257 --d 80 --dtype bf16

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
    ap.add_argument("kind", choices=["conv", "gemm", "attention"])
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
    a = ap.parse_args(argv)
    dt = torch.float16 if a.dtype == "fp16" else torch.bfloat16
    dev = "cuda"
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


if __name__ == "__main__":
    sys.exit(main())
