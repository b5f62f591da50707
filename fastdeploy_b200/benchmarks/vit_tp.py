"""ViT-H/14 classification (632 M parameters, 32 layers, hidden 1280, 16 heads, MLP 5120), 224x224 images, batch
256, tensor-parallel over the N GPUs of one box with the fused GEMM + collective kernels (all-gather -> column
GEMM, row GEMM -> reduce-scatter). The reference has no tensor parallelism; the library baseline beside the
number is NCCL + cuBLAS + flash SDPA in the same sharding, and the roofline is the slower of the tensor-core time
at the measured GEMM peak and the bytes over NVLink at the measured link bandwidth."""
from __future__ import annotations

from .common import ClockSampler, Context, median, physical_gpu_index, spread


def run(ctx: Context, args) -> dict:
    torch = ctx.torch
    from fastdeploy_b200.parallel.bench_vit import _LibraryBaseline
    from fastdeploy_b200.parallel.comm import Communicator
    from fastdeploy_b200.parallel.vit import VIT_SIZES, TensorParallelViT, random_vit_weights
    dev, world = ctx.dev, ctx.world
    size, image, B = "huge14", 224, args.batch or 256
    dtype_name = args.dtype or "bf16"
    dtype = torch.bfloat16
    cfg = VIT_SIZES[size]
    T = (image // cfg["patch"]) ** 2 + 1
    m_pad = (B * T + world * 128 - 1) // (world * 128) * (world * 128)
    heap = (2 if dtype_name == "fp8" else 1) * 4 * m_pad * cfg["hidden"] * 2 + (64 << 20)
    comm = Communicator(heap_bytes=heap)
    w = random_vit_weights(cfg, image, 1000, seed=0)
    g = torch.Generator(device="cpu").manual_seed(1)
    host_sets = [torch.rand(B, 3, image, image, generator=g).to(dtype).pin_memory() for _ in range(2)]
    dev_sets = [t.to(dev) for t in host_sets]
    model = TensorParallelViT(comm, w, cfg, batch=B, image=image, dtype=dtype)
    if dtype_name == "fp8":
        # post-training quantisation: static activation scales from one calibration batch of the 16-bit model
        scales = model.calibrate(dev_sets[0])
        del model
        torch.cuda.empty_cache()
        model = TensorParallelViT(comm, w, cfg, batch=B, image=image, dtype=dtype, precision="fp8", act_scales=scales,
                                  name="tpvit8")
    sampler = ClockSampler(physical_gpu_index(ctx.local_rank))
    sampler.start()

    def dev_steps(n):
        for i in range(n):
            model.forward(dev_sets[i & 1])
    sampler.wait_ready()
    warm = max(args.warmup, 3)
    dev_steps(warm)
    comm.check("tp vit warm-up")
    ctx.barrier()
    sampler.rows.clear()
    dev_ms = ctx.time_blocks(dev_steps, args.steps, args.repeats)
    enc_ms = ctx.time_blocks(lambda n: [model.encoder() for _ in range(n)], args.steps, 3)
    comm.check("tp vit timed")
    stage = torch.empty_like(dev_sets[0])
    probs_host = torch.empty(B, 1000, dtype=torch.float32).pin_memory()
    acc = [0.0]

    def e2e_steps(n):
        for i in range(n):
            stage.copy_(host_sets[i & 1], non_blocking=True)
            probs = model.forward(stage)
            probs_host.copy_(probs, non_blocking=True)
            torch.cuda.current_stream().synchronize()
            acc[0] += float(probs_host[0, 0])
    e2e_steps(warm)
    e2e_ms = ctx.time_blocks(e2e_steps, args.steps, args.repeats)
    comm.check("tp vit e2e")
    base = _LibraryBaseline(w, cfg, B, image, dtype, ctx.rank, world, dev, 1e-6)
    with torch.no_grad():
        lib_ms = ctx.time_blocks(lambda n: [base.encoder() for _ in range(n)], args.steps, 3)
    clocks = sampler.stop()
    ms, enc, lib = median(dev_ms) / args.steps, median(enc_ms) / args.steps, median(lib_ms) / args.steps
    fl = model.flops()
    nv = 4.0 * len(model.layers) * (world - 1) / world * model.M * cfg["hidden"] * 2
    roof = max(fl / world / 1404.3e12, nv / 770e9) * 1e3
    out = {
        "metric": "images/sec ViT-H/14 tensor-parallel (device-timed)", "value": round(B / ms * 1e3, 1),
        "unit": "images/s", "n_gpus": world, "steps": args.steps, "warmup": warm, "ms_per_step": round(ms, 3),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": dtype_name, "data": "synthetic",
        "config": {"model": "ViT-H/14 224x224, 632M parameters, random-init weights", "global_batch": B,
                   "seq_len": T, "parallelism": f"tp{world}",
                   "l2_policy": "activations of one layer (168 MB at batch 256) exceed L2; two alternating image sets",
                   "timing": f"median of {args.repeats} blocks of {args.steps} steps, CUDA events, max over ranks",
                   "baseline_ref": "no tensor parallelism in the reference; library baseline = NCCL + cuBLAS + flash SDPA"},
        "block_ms": spread(dev_ms),
        "encoder_ms": round(enc, 3), "library_encoder_ms": round(lib, 3),
        "encoder_vs_library": round(lib / enc, 3),
        "roofline_ms": round(roof, 3), "roofline_frac": round(roof / enc, 3),
        "roofline_denominators": "1404.3 TFLOP/s sustained cuBLAS bf16 (measured), 770 GB/s peer copy per direction (measured)",
        "e2e": {"value": round(B / (median(e2e_ms) / args.steps) * 1e3, 1), "unit": "images/s",
                "h2d_bytes_per_step": int(host_sets[0].numel() * 2), "d2h_bytes_per_step": int(B * 1000 * 4),
                "ms_per_step": round(median(e2e_ms) / args.steps, 3), "block_ms": spread(e2e_ms),
                "what": "pinned images -> device, TensorParallelViT.forward, class probabilities -> pinned host"},
        "gpu_launches": int(model.launches_per_forward * args.steps), "clocks": clocks, "cpu_affinity": ctx.affinity,
        "impl": "ours",
    }
    comm.close()
    return out
