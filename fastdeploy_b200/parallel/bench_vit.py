"""Tensor-parallel ViT check + benchmark, one process per GPU:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port 29541 \
        -m fastdeploy_b200.parallel.bench_vit --size huge14 --batch 256 --steps 10 --warmup 3

(or plain ``python -m fastdeploy_b200.parallel.bench_vit`` for one GPU). ``--check`` compares the class
probabilities with the fp32 PyTorch forward of the same weights. Timing is on the device (CUDA events,
maximum over ranks). The library baseline printed beside it is the same network written with torch ops
(cuBLAS GEMMs, flash SDPA) and NCCL all-gather / reduce-scatter in the same sequence-sharded layout.
Rank 0 prints one line that starts with ``TPVIT``.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

from .comm import Communicator
from .vit import VIT_SIZES, TensorParallelViT, random_vit_weights, vit_reference


def _timed(fn, steps, warmup, world):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / steps], device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t[0])


class _LibraryBaseline:
    """Same sharding, library kernels only: NCCL collectives + cuBLAS + flash SDPA."""

    def __init__(self, w, cfg, batch, image, dtype, rank, world, dev, eps):
        H, NH, F = cfg["hidden"], cfg["heads"], cfg["mlp"]
        self.cfg, self.B, self.T, self.eps = cfg, batch, (image // cfg["patch"]) ** 2 + 1, eps
        self.rank, self.world, self.dt = rank, world, dtype
        D = H // NH
        hd, fl = H // world, F // world
        self.hl, self.D = NH // world, D
        unit = world * 128
        self.M = (batch * self.T + unit - 1) // unit * unit
        self.rows = self.M // world
        sl, fs = slice(rank * hd, (rank + 1) * hd), slice(rank * fl, (rank + 1) * fl)
        self.layers = []
        for l in range(cfg["layers"]):
            p = f"blocks.{l}."
            g = lambda k: w[p + k].to(dev).to(dtype)
            self.layers.append(dict(
                ln1=(g("ln1_g"), g("ln1_b")), ln2=(g("ln2_g"), g("ln2_b")),
                wqkv=torch.cat([g("q_w")[sl], g("k_w")[sl], g("v_w")[sl]]),
                bqkv=torch.cat([g("q_b")[sl], g("k_b")[sl], g("v_b")[sl]]),
                wproj=g("proj_w")[:, sl].contiguous(), bproj=g("proj_b"),
                w1=g("fc1_w")[fs].contiguous(), b1=g("fc1_b")[fs].contiguous(),
                w2=g("fc2_w")[:, fs].contiguous(), b2=g("fc2_b")))
        self.x = torch.randn(self.rows, H, device=dev).to(dtype)
        self.full = torch.empty(self.M, H, dtype=dtype, device=dev)
        self.rs = torch.empty(self.rows, H, dtype=dtype, device=dev)

    def _ag(self, h):
        if self.world == 1:
            return h
        dist.all_gather_into_tensor(self.full, h)
        return self.full

    def _rs(self, part):
        if self.world == 1:
            return part
        dist.reduce_scatter_tensor(self.rs, part)
        return self.rs

    def encoder(self):
        import torch.nn.functional as Fn
        x, H, B, T = self.x, self.cfg["hidden"], self.B, self.T
        hd = self.hl * self.D
        for L in self.layers:
            h = self._ag(Fn.layer_norm(x, (H,), *L["ln1"], self.eps))
            qkv = Fn.linear(h, L["wqkv"], L["bqkv"])
            q, k, v = (qkv[:B * T, i * hd:(i + 1) * hd].view(B, T, self.hl, self.D).transpose(1, 2) for i in range(3))
            a = Fn.scaled_dot_product_attention(q, k, v).transpose(1, 2).reshape(B * T, hd)
            if self.M > B * T:
                a = Fn.pad(a, (0, 0, 0, self.M - B * T))
            x = x + self._rs(Fn.linear(a, L["wproj"])) + L["bproj"]
            h = self._ag(Fn.layer_norm(x, (H,), *L["ln2"], self.eps))
            x = x + self._rs(Fn.linear(Fn.gelu(Fn.linear(h, L["w1"], L["b1"])), L["w2"])) + L["b2"]
        return x


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--size", default="huge14", choices=sorted(VIT_SIZES))
    ap.add_argument("--batch", type=int, default=256)
    ap.add_argument("--image", type=int, default=224)
    ap.add_argument("--classes", type=int, default=1000)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--check", action="store_true")
    ap.add_argument("--no-baseline", action="store_true")
    ap.add_argument("--breakdown", action="store_true", help="one rank only: device time of each launch kind")
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "fp16", "fp8"],
                    help="fp8: e4m3 operands in the four linears of every block (bf16 elsewhere), static activation "
                         "scales calibrated on the first batch")
    a = ap.parse_args(argv)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    dtype = torch.float16 if a.dtype == "fp16" else torch.bfloat16
    cfg = VIT_SIZES[a.size]
    T = (a.image // cfg["patch"]) ** 2 + 1
    m_pad = (a.batch * T + world * 128 - 1) // (world * 128) * (world * 128)
    heap = (2 if a.dtype == "fp8" else 1) * (2 * m_pad * cfg["hidden"] * 2 + 2 * m_pad * cfg["hidden"] * 2) + (64 << 20)
    comm = Communicator(heap_bytes=heap)
    w = random_vit_weights(cfg, a.image, a.classes, seed=0)
    g = torch.Generator(device="cpu").manual_seed(1)
    images = torch.rand(a.batch, 3, a.image, a.image, generator=g).to(dev).to(dtype)
    model = TensorParallelViT(comm, w, cfg, batch=a.batch, image=a.image, dtype=dtype)
    if a.dtype == "fp8":
        scales = model.calibrate(images)
        comm.check("tp vit calibration")
        del model
        model = TensorParallelViT(comm, w, cfg, batch=a.batch, image=a.image, dtype=dtype, precision="fp8",
                                  act_scales=scales, name="tpvit8")
    out = {"world": world, "size": a.size, "batch": a.batch, "tokens": a.batch * T, "dtype": a.dtype}
    probs = model.forward(images)
    comm.check("tp vit forward")
    if a.check:
        ref = vit_reference(w, cfg, images.float())
        out["max_abs_err"] = float((probs - ref).abs().max())
        out["top1_agree"] = float((probs.argmax(-1) == ref.argmax(-1)).float().mean())
        out["ref_max_prob"] = float(ref.max())
    if a.steps > 0:
        ms = _timed(lambda: model.forward(images), a.steps, a.warmup, world)
        enc = _timed(model.encoder, a.steps, a.warmup, world)
        comm.check("tp vit timed")
        fl = model.flops()
        out.update(forward_ms=ms, encoder_ms=enc, images_per_s=a.batch / ms * 1e3,
                   encoder_tflops_per_gpu=fl / world / enc / 1e9,
                   launches_per_forward=model.launches_per_forward)
        # roofline of the encoder per GPU: tensor-core time at the measured sustained cuBLAS bf16 rate against
        # the bytes each GPU must pull / push over NVLink (4 collectives per layer) at 770 GB/s per direction
        nv = 4.0 * len(model.layers) * (world - 1) / world * model.M * cfg["hidden"] * 2
        out["roofline_ms"] = max(fl / world / 1404.3e12, nv / 770e9) * 1e3
        out["roofline_frac"] = out["roofline_ms"] / enc
        if a.breakdown and world > 1:
            # every rank runs the same launch sequence, so each piece synchronises itself through the device
            # barriers / counters it contains; times are device time, max over ranks
            lay = model.layers[0]
            nxt = model.layers[1]["ln1_gb"] + (model.shard[0],) + ((1.0 / model.layers[1]["scales"][0],) if model.fp8 else ())
            ln2 = lay["ln2_gb"] + (model.shard[1],) + ((1.0 / lay["scales"][2],) if model.fp8 else ())
            parts = {
                "barrier+allgather_qkv": lambda: (comm.barrier(), lay["qkv"].launch()),
                "attention": model.attn.launch,
                "proj_reducescatter+reduce_ln": lambda: (lay["proj"].launch(), model._reduce_into_residual(0, lay["proj"], lay["proj_b"], ln2)),
                "barrier+allgather_fc1": lambda: (comm.barrier(), lay["fc1"].launch()),
                "fc2_reducescatter+reduce_ln": lambda: (lay["fc2"].launch(), model._reduce_into_residual(1, lay["fc2"], lay["fc2_b"], nxt)),
                "barrier": comm.barrier,
            }
            out["breakdown_ms"] = {k: round(_timed(f, a.steps, a.warmup, world), 4) for k, f in parts.items()}
            comm.check("tp vit breakdown")
        if a.breakdown and world == 1:
            lay = model.layers[0]
            parts = {"ln": lay["ln1"].launch, "qkv": lay["qkv"].launch, "fc1": lay["fc1"].launch,
                     "proj": lay["proj"].launch, "fc2": lay["fc2"].launch, "barrier": comm.barrier,
                     "reduce": lambda: (model.counters[0].fill_(1 << 30), model._reduce_into_residual(0, lay["proj"], lay["proj_b"], lay["ln2_gb"] + (model.shard[1],)))}
            parts.update({"attn_" + op.name: op.launch for op in model.attn.ops})
            out["breakdown_ms"] = {k: round(_timed(f, a.steps, a.warmup, 1), 4) for k, f in parts.items()}
            model.counters[0].zero_(); model.counters[1].zero_(); model.targets = [0, 0]
        if not a.no_baseline:
            base = _LibraryBaseline(w, cfg, a.batch, a.image, dtype, rank, world, dev, 1e-6)
            with torch.no_grad():
                out["library_encoder_ms"] = _timed(base.encoder, a.steps, a.warmup, world)
    if rank == 0:
        print("TPVIT " + json.dumps(out), flush=True)
    comm.close()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
