"""Per-step timing of a launch plan: which layer runs which kernel variant, and how fast.

    python -m fastdeploy_b200.utils.layer_profile --model ppyoloe --variant l --batch 32 --image 640 \
        --peak-tflops 1404.3 --peak-gbs 6545 --out table.md

Every step of the plan (one native launch each) is timed alone with CUDA events: ``--iters`` launches,
each preceded by a write of a buffer larger than L2 so that a layer never finds its own input from the
previous iteration in cache, and the median is reported. For tensor-core steps the table gives the shape,
the kernel variant and tile the planner chose, TFLOP/s and the fraction of ``--peak-tflops``; for the rest
the time alone. The sum of the per-step times is a little above the time of the captured plan (no overlap
between the tail of one kernel and the head of the next when each is timed alone).

The counterpart in the reference is the per-backend profile loop (fastdeploy/benchmark/benchmark.h:21-85),
which can only time the whole engine call.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import tempfile


def build_model(args):
    import fastdeploy_b200 as fd
    fd.set_logger(False, True)
    opt = fd.RuntimeOption()
    opt.use_gpu(0)
    if args.dtype == "bf16":
        opt.native_option.precision = "bf16"
    d = args.model_dir or tempfile.mkdtemp(prefix=f"fdb200_{args.model}_")
    if args.model == "ppyoloe":
        from ..models.ppyoloe import write_ppyoloe
        paths = write_ppyoloe(d, args.variant, image=args.image, num_classes=80, seed=0, score_threshold=0.01,
                              nms_threshold=0.6, nms_top_k=1000, keep_top_k=100)
        rt = fd.Runtime(_opt_with_model(opt, paths["model"], paths["params"]))
        shapes = {}
        for vi in rt.graph.inputs:
            shapes[vi.name] = [args.batch, 3, args.image, args.image] if vi.name == "image" else [args.batch, 2]
        return rt, shapes
    if args.model == "resnet50":
        from ..models.resnet import resnet50_onnx
        path = os.path.join(d, "resnet50.onnx")
        resnet50_onnx(path)
        opt.set_model_path(path, "", fd.ModelFormat.ONNX)
        rt = fd.Runtime(opt)
        return rt, {rt.graph.inputs[0].name: [args.batch, 3, args.image, args.image]}
    if args.model == "ernie":
        # ERNIE-3.0-base sequence classification, bf16; --packed runs the padding-free plan on sequences with lengths
        # uniform in 16..512 (the bucket that holds them), otherwise the plan padded to 512 tokens
        import numpy as np
        from ..models.ernie import SIZES, write_ernie
        if not os.path.exists(os.path.join(d, "model.pdiparams")):
            write_ernie(d, args.variant if args.variant in SIZES else "base", "seq_cls", seed=0, vocab=False)
        opt.native_option.precision = "bf16"
        rt = fd.Runtime(_opt_with_model(opt, os.path.join(d, "model.pdmodel"), os.path.join(d, "model.pdiparams")))
        names = [vi.name for vi in rt.graph.inputs]
        if not args.packed:
            return rt, {n: [args.batch, 512] for n in names}
        from ..text.packed import PackedEncoder
        rng = np.random.default_rng(99)
        lens = rng.integers(16, 513, args.batch)
        seqs = [(rng.integers(1, 40000, n), np.zeros(n, np.int64)) for n in lens]
        enc = PackedEncoder(rt, max_tokens=args.batch * 512, max_seqs=args.batch, max_len=512,
                            token_buckets=range(2048, args.batch * 512 + 1, 2048))
        bk, feeds, _, _ = enc.pack(seqs)
        enc.launch(bk, feeds)
        print(f"packed: {int(lens.sum())} tokens of {args.batch} sequences in a bucket of {bk.rows} rows")
        return rt, bk.plan
    raise SystemExit(f"unknown model {args.model}")


def _opt_with_model(opt, model, params):
    opt.set_model_path(model, params)
    return opt


def conv_flops(meta) -> float:
    n, h, w, cin = meta["in_shape"]
    ho, wo = meta["out_hw"]
    kh, kw = meta["kernel"]
    return 2.0 * n * ho * wo * meta["cout"] * meta["cin_logical"] * kh * kw


def main(argv=None) -> int:
    import torch
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="ppyoloe", choices=["ppyoloe", "resnet50", "ernie"])
    ap.add_argument("--packed", action="store_true", help="ernie: the padding-free plan instead of the padded one")
    ap.add_argument("--variant", default="l")
    ap.add_argument("--batch", type=int, default=32)
    ap.add_argument("--image", type=int, default=640)
    ap.add_argument("--dtype", default="fp16")
    ap.add_argument("--iters", type=int, default=7)
    ap.add_argument("--peak-tflops", type=float, default=0.0, help="measured dense 16-bit GEMM peak of this GPU")
    ap.add_argument("--peak-gbs", type=float, default=0.0, help="measured copy bandwidth of this GPU")
    ap.add_argument("--model-dir", default="")
    ap.add_argument("--out", default="")
    ap.add_argument("--top", type=int, default=0, help="only print the N slowest steps")
    a = ap.parse_args(argv)

    rt, shapes = build_model(a)
    plan = rt.plan_for_shapes(shapes) if isinstance(shapes, dict) else shapes
    dev = rt.device
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    rows = []
    with torch.cuda.device(dev):
        # whole plan, as it runs in production (CUDA graph replay)
        for _ in range(3):
            plan.run()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize(dev)
        e0.record()
        for _ in range(10):
            plan.run()
        e1.record()
        torch.cuda.synchronize(dev)
        plan_ms = e0.elapsed_time(e1) / 10
        for idx, st in enumerate(plan.steps):
            times = []
            for _ in range(a.iters):
                flush.fill_(1)
                s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                s.record()
                st.fn()
                e.record()
                e.synchronize()
                times.append(s.elapsed_time(e))
            times.sort()
            ms = times[len(times) // 2]
            meta = getattr(st.native, "meta", None) if st.native is not None else None
            row = {"idx": idx, "name": st.name, "ms": ms, "kind": "py" if st.native is None else "native"}
            if meta is not None:
                info = st.native.info()
                fl = conv_flops(meta)
                row.update(shape=f'{meta["in_shape"][0]}x{meta["in_shape"][1]}x{meta["in_shape"][2]}x{meta["cin_logical"]}'
                                 f'->{meta["cout"]} k{meta["kernel"][0]} s{meta["stride"]}',
                           variant={0: "generic", 1: "halo", 2: "halo-resident", 3: "pair", 4: "halo-pair",
                                    5: "halo-pair-resident"}.get(info["variant"], "?"),
                           tile=f'{info["tile_w"]}x{info["tile_h"]}xN{info["block_n"]}', grid=info["grid"],
                           gflop=fl / 1e9, tflops=fl / ms / 1e9, bytes=meta["bytes"])
            rows.append(row)
    plan.status.check("layer profile")
    total = sum(r["ms"] for r in rows)
    conv_ms = sum(r["ms"] for r in rows if "tflops" in r)
    conv_fl = sum(r["gflop"] for r in rows if "tflops" in r)
    lines = [f"plan: {len(plan.steps)} steps, graph replay {plan_ms:.3f} ms per batch; sum of steps timed alone "
             f"{total:.3f} ms; tensor-core steps {conv_ms:.3f} ms for {conv_fl / 1e3:.3f} TFLOP = "
             f"{conv_fl / conv_ms:.0f} TFLOP/s" + (f" = {conv_fl / conv_ms / a.peak_tflops:.2f} of {a.peak_tflops} (measured)"
                                                   if a.peak_tflops else ""), "",
             "| # | step | shape | variant | tile | grid | ms | TFLOP/s | of peak | GB/s |", "|---|---|---|---|---|---|---|---|---|---|"]
    show = sorted(rows, key=lambda r: -r["ms"])[:a.top] if a.top else rows
    for r in show:
        if "tflops" in r:
            frac = f'{r["tflops"] / a.peak_tflops:.2f}' if a.peak_tflops else ""
            lines.append(f'| {r["idx"]} | {r["name"]} | {r["shape"]} | {r["variant"]} | {r["tile"]} | {r["grid"]} | '
                         f'{r["ms"]:.4f} | {r["tflops"]:.0f} | {frac} | {r["bytes"] / r["ms"] / 1e6:.0f} |')
        else:
            lines.append(f'| {r["idx"]} | {r["name"]} |  | {r["kind"]} |  |  | {r["ms"]:.4f} |  |  |  |')
    kinds = {}
    for r in rows:
        k = r["name"].split(":")[0].split("(")[0]
        kinds.setdefault(k, [0, 0.0])
        kinds[k][0] += 1
        kinds[k][1] += r["ms"]
    lines += ["", "| kind | steps | ms | share |", "|---|---|---|---|"]
    for k, (cnt, ms) in sorted(kinds.items(), key=lambda kv: -kv[1][1]):
        lines.append(f"| {k} | {cnt} | {ms:.3f} | {100 * ms / total:.1f} % |")
    text = "\n".join(lines)
    print(text)
    if a.out:
        with open(a.out, "w") as f:
            f.write(text + "\n")
        with open(os.path.splitext(a.out)[0] + ".json", "w") as f:
            json.dump({"plan_ms": plan_ms, "rows": rows}, f)
    return 0


if __name__ == "__main__":
    sys.exit(main())
