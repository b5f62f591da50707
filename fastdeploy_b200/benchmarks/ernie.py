"""ERNIE-3.0-base sequence classification, bf16, batch 64 per GPU, token ids uniform, lengths uniform in
16..512 padded to 512 (the mask is derived from the pad id inside the graph), data-parallel. The reference's
driver is benchmark/python/benchmark_ernie_seq_cls.py:133-274 (host timers around ``runtime.infer``)."""
from __future__ import annotations

import os
import tempfile

from .common import ClockSampler, Context, median, physical_gpu_index, spread


def make_batch(rng, batch: int, seq: int, vocab: int):
    import numpy as np
    lens = rng.integers(16, seq + 1, batch)
    ids = np.zeros((batch, seq), np.int64)
    for i, n in enumerate(lens):
        ids[i, :n] = rng.integers(1, vocab, n)
    return ids, np.zeros((batch, seq), np.int64), lens


def run(ctx: Context, args) -> dict:
    import numpy as np
    torch = ctx.torch
    import fastdeploy_b200 as fd
    from fastdeploy_b200.models.ernie import SIZES, write_ernie
    fd.set_logger(False, True)
    dev = ctx.dev
    size = "base"
    model_dir = args.model_dir or os.path.join(tempfile.gettempdir(), f"fdb200_ernie_{size}_seqcls")
    if ctx.rank == 0 and not os.path.exists(os.path.join(model_dir, "model.pdiparams")):
        write_ernie(model_dir, size, "seq_cls", seed=0, vocab=False)
    ctx.barrier()
    opt = fd.RuntimeOption()
    opt.use_gpu(ctx.local_rank)
    opt.native_option.precision = "bf16"
    opt.set_model_path(os.path.join(model_dir, "model.pdmodel"), os.path.join(model_dir, "model.pdiparams"))
    rt = fd.Runtime(opt)
    B, S = args.batch or 64, 512
    rng = np.random.default_rng(99 + ctx.rank)
    names = [vi.name for vi in rt.graph.inputs]
    host_sets, dev_sets, tokens = [], [], 0
    for _ in range(4):
        ids, types, lens = make_batch(rng, B, S, SIZES[size]["vocab"])
        tokens += int(lens.sum())
        hs = {names[0]: torch.from_numpy(ids).pin_memory(), names[1]: torch.from_numpy(types).pin_memory()}
        host_sets.append({k: v.numpy() for k, v in hs.items()})
        dev_sets.append({k: v.to(dev) for k, v in hs.items()})
    sampler = ClockSampler(physical_gpu_index(ctx.local_rank))
    sampler.start()
    plan = rt.plan_for_shapes({n: [B, S] for n in names})
    flush = torch.empty(192 << 20, dtype=torch.uint8, device=dev)      # larger than L2: written between steps

    def dev_steps(n):
        for i in range(n):
            flush.fill_(i & 1)
            for k, v in dev_sets[i % 4].items():
                plan.inputs[k].t.copy_(v)
            plan.run()
            rt.gpu_launches += plan.native_kernel_launches
    sampler.wait_ready()
    warm = max(args.warmup, 3)
    dev_steps(warm)
    plan.status.check("ernie warm-up")
    ctx.barrier()
    sampler.rows.clear()
    l0 = rt.gpu_launches
    dev_ms = ctx.time_blocks(dev_steps, args.steps, args.repeats)
    launches = (rt.gpu_launches - l0) // args.repeats
    # the flush itself, timed alone, is taken out of the step time
    def flush_steps(n):
        for i in range(n):
            flush.fill_(i & 1)
    flush_ms = median(ctx.time_blocks(flush_steps, args.steps, 3))
    out_sum = [0.0]

    def e2e_steps(n):
        for i in range(n):
            logits = rt.infer(host_sets[i % 4])[0]
            out_sum[0] += float(logits[0, 0])
    e2e_steps(warm)
    e2e_ms = ctx.time_blocks(e2e_steps, args.steps, args.repeats)
    # ---- padding-free mode: the same sequences back to back, one plan per bucket of packed rows
    from fastdeploy_b200.text.packed import PackedEncoder
    enc = PackedEncoder(rt, max_tokens=B * S, max_seqs=B, max_len=S, token_buckets=range(4096, B * S + 1, 2048))
    seq_sets, packed_dev = [], []
    for hs in host_sets:
        ids, types = hs[names[0]], hs[names[1]]
        lens = (ids != 0).sum(1)
        seqs = [(ids[i, :n], types[i, :n]) for i, n in enumerate(lens)]
        seq_sets.append(seqs)
        bk, feeds, _, _ = enc.pack(seqs)
        packed_dev.append((bk, {k: torch.from_numpy(np.ascontiguousarray(v)).to(dev) for k, v in feeds.items()}))

    def packed_steps(n):
        for i in range(n):
            flush.fill_(i & 1)
            bk, feeds = packed_dev[i % 4]
            for k, v in feeds.items():
                bk.plan.inputs[k].t.copy_(v.reshape(bk.plan.inputs[k].t.shape))
            bk.plan.run()
            rt.gpu_launches += bk.plan.native_kernel_launches
    packed_steps(warm)
    for bk, _ in packed_dev:
        bk.plan.status.check("packed warm-up")
    # the packed plans return the padded plans' logits
    ref_logits = rt.infer(host_sets[0])[0]
    got_logits = enc.infer(seq_sets[0])[0]
    packed_err = float(np.abs(got_logits - ref_logits).max())
    ctx.barrier()
    l1 = rt.gpu_launches
    packed_ms = ctx.time_blocks(packed_steps, args.steps, args.repeats)
    packed_launches = (rt.gpu_launches - l1) // args.repeats

    def packed_e2e_steps(n):
        for i in range(n):
            logits = enc.infer(seq_sets[i % 4])[0]
            out_sum[0] += float(logits[0, 0])
    packed_e2e_steps(warm)
    packed_e2e_ms = ctx.time_blocks(packed_e2e_steps, args.steps, args.repeats)
    clocks = sampler.stop()
    ms_packed = median(packed_ms) - flush_ms
    ms_packed_e2e = median(packed_e2e_ms)
    packed_rows = [bk.rows for bk, _ in packed_dev]
    ms_dev = median(dev_ms) - flush_ms
    ms_e2e = median(e2e_ms)
    seqs = B * ctx.world * args.steps
    py_steps = [s.name for s in plan.steps if s.native is None]
    padded = {"value": round(seqs / (ms_dev / 1e3), 1), "unit": "sequences/s", "ms_per_step": round(ms_dev / args.steps, 3),
              "block_ms": spread(dev_ms), "e2e_value": round(seqs / (ms_e2e / 1e3), 1),
              "e2e_ms_per_step": round(ms_e2e / args.steps, 3), "gpu_launches": int(launches),
              "plan_steps": len(plan.steps), "h2d_bytes_per_step": int(2 * B * S * 8),
              "what": "every sequence padded to 512 tokens, additive mask from the pad id (Runtime.infer for the end-to-end "
                      "figure)"}
    packed_plan = packed_dev[0][0].plan
    h2d = int(sum(v.numel() * v.element_size() for v in packed_dev[0][1].values()))
    return {
        "metric": "sequences/sec ERNIE-3.0-base seq-cls (device-timed)", "value": round(seqs / (ms_packed / 1e3), 1),
        "unit": "sequences/s", "n_gpus": ctx.world, "steps": args.steps, "warmup": warm,
        "ms_per_step": round(ms_packed / args.steps, 3), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": {"model": "ERNIE-3.0-base (12 layers, hidden 768, 12 heads, vocab 40000) seq-cls, random-init weights",
                   "global_batch": B * ctx.world, "seq_len": S, "parallelism": f"dp{ctx.world}",
                   "lengths": "uniform 16..512",
                   "execution": "padding-free: sequences packed back to back (starts aligned to 8 rows), attention per "
                                "sequence from device-side starts / lengths, first-token gather; one plan per bucket of "
                                "2048 packed rows; logits equal the padded plan's (difference below)",
                   "real_tokens_per_step": tokens // 4, "bucket_rows": packed_rows,
                   "max_abs_diff_vs_padded_logits": packed_err,
                   "l2_policy": "192 MB written between steps (its own time, measured alone, is subtracted)",
                   "timing": f"median of {args.repeats} blocks of {args.steps} steps, CUDA events, max over ranks",
                   "baseline_ref": "the reference publishes no ERNIE latency"},
        "block_ms": spread(packed_ms),
        "e2e": {"value": round(seqs / (ms_packed_e2e / 1e3), 1), "unit": "sequences/s",
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": int(B * 2 * 4 + 4),
                "ms_per_step": round(ms_packed_e2e / args.steps, 3), "block_ms": spread(packed_e2e_ms),
                "what": "PackedEncoder.infer on lists of int64 id arrays: packing on the host, pinned staging, logits "
                        "read back every step"},
        "gpu_launches": int(packed_launches), "plan_steps": len(packed_plan.steps),
        "non_native_steps": [s.name for s in packed_plan.steps if s.native is None] + py_steps,
        "clocks": clocks, "cpu_affinity": ctx.affinity, "impl": "ours", "padded": padded,
    }
