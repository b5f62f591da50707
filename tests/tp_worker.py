"""Worker of the multi-GPU tests: ``python -m torch.distributed.run --nproc-per-node N tests/tp_worker.py``.
Checks the peer-memory collectives and the fused tensor-parallel GEMMs against NCCL + torch fp32
references and prints one JSON line with device-timed comparisons (max over ranks)."""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def timed(fn, iters=10, warm=3):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / iters], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t[0])


def main():
    rank = int(os.environ["RANK"])
    local = int(os.environ["LOCAL_RANK"])
    world = int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from fastdeploy_b200.parallel import ColumnParallelLinear, Communicator, RowParallelLinear, TensorParallelMLP
    comm = Communicator(heap_bytes=1 << 30)
    out = {"world": world}
    dt = torch.bfloat16
    g = torch.Generator(device="cpu").manual_seed(100 + rank)

    # ---- collectives vs NCCL
    x = (torch.randn(world * 256, 512, generator=g) * 0.5).to(dt).to(dev)
    ref = x.float().clone()
    dist.all_reduce(ref)
    got = comm.all_reduce(x)
    out["allreduce_err"] = float((got.float() - ref).abs().max())
    rs = comm.reduce_scatter(x)
    out["reducescatter_err"] = float((rs.float() - ref[rank * 256:(rank + 1) * 256]).abs().max())
    ag = comm.all_gather_tensor(x[:256].contiguous())
    ref_ag = [torch.empty(256, 512, dtype=dt, device=dev) for _ in range(world)]
    dist.all_gather(ref_ag, x[:256].contiguous())
    out["allgather_err"] = float((ag.float() - torch.cat(ref_ag).float()).abs().max())

    # ---- all-gather -> GEMM (column parallel): M x K times (N / world) x K
    mpr = int(os.environ.get("TP_M_PER_RANK", "1024"))
    M, K, N = world * mpr, 1280, 5120
    gw = torch.Generator(device="cpu").manual_seed(7)
    w_full = torch.randn(N, K, generator=gw) * 0.03
    b_full = torch.randn(N, generator=gw)
    nl = N // world
    col = ColumnParallelLinear(comm, M, K, w_full[rank * nl:(rank + 1) * nl], b_full[rank * nl:(rank + 1) * nl],
                               act="gelu", dtype=dt)
    x_shard = (torch.randn(M // world, K, generator=g) * 0.5).to(dt).to(dev)
    col.input_tensor().copy_(x_shard)
    y = col.forward()
    torch.cuda.synchronize()
    xs = [torch.empty_like(x_shard) for _ in range(world)]
    dist.all_gather(xs, x_shard)
    x_full = torch.cat(xs).float()
    ref_y = torch.nn.functional.gelu(x_full @ w_full[rank * nl:(rank + 1) * nl].to(dev).to(dt).float().T
                                     + b_full[rank * nl:(rank + 1) * nl].to(dev))
    out["col_err"] = float((y.float() - ref_y).abs().max() / ref_y.abs().max())

    def col_baseline():
        dist.all_gather(xs, x_shard)
        xf = torch.cat(xs)
        return torch.nn.functional.gelu(torch.nn.functional.linear(xf, wl, bl), approximate="none")
    wl = w_full[rank * nl:(rank + 1) * nl].to(dev).to(dt)
    bl = b_full[rank * nl:(rank + 1) * nl].to(dev).to(dt)
    out["col_fused_ms"] = timed(col.forward)
    out["col_nccl_torch_ms"] = timed(col_baseline)

    # ---- GEMM -> reduce-scatter (row parallel): M x (K / world) times N x (K / world)
    K2, N2 = 5120, 1280
    kl = K2 // world
    w2 = torch.randn(N2, K2, generator=gw) * 0.03
    b2 = torch.randn(N2, generator=gw)
    row = RowParallelLinear(comm, M, kl, N2, w2[:, rank * kl:(rank + 1) * kl], b2, dtype=dt)
    assert kl == nl
    gx = torch.Generator(device="cpu").manual_seed(11)
    x2_full = (torch.randn(M, K2, generator=gx) * 0.5).to(dt)
    row.input_tensor().copy_(x2_full[:, rank * kl:(rank + 1) * kl].to(dev))
    y2 = row.forward()
    torch.cuda.synchronize()
    ref2 = x2_full.float().to(dev) @ w2.to(dt).float().to(dev).T + b2.to(dev)
    rows = M // world
    out["row_err"] = float((y2.float() - ref2[rank * rows:(rank + 1) * rows]).abs().max() / ref2.abs().max())
    w2l = w2[:, rank * kl:(rank + 1) * kl].to(dev).to(dt)
    x2l = row.input_tensor()
    rs_out = torch.empty(rows, N2, dtype=dt, device=dev)

    def row_baseline():
        part = torch.nn.functional.linear(x2l, w2l)
        dist.reduce_scatter_tensor(rs_out, part)
        return rs_out
    out["row_fused_ms"] = timed(row.forward)
    out["row_nccl_torch_ms"] = timed(row_baseline)
    # ---- whole feed-forward block (ViT-H sizes: hidden 1280, ffn 5120), row shards in and out
    mlp = TensorParallelMLP(comm, M, K, N, w_full, b_full, w2, b2, dtype=dt)
    mlp.input_tensor().copy_(x_shard)
    ym = mlp.forward()
    torch.cuda.synchronize()
    h_ref = torch.nn.functional.gelu(x_full @ w_full.to(dev).to(dt).float().T + b_full.to(dev)).to(dt).float()
    ref_m = h_ref @ w2.to(dev).to(dt).float().T + b2.to(dev)
    out["mlp_err"] = float((ym.float() - ref_m[rank * rows:(rank + 1) * rows]).abs().max() / ref_m.abs().max())
    w1l, b1l = wl, bl

    def mlp_baseline():
        dist.all_gather(xs, x_shard)
        h = torch.nn.functional.gelu(torch.nn.functional.linear(torch.cat(xs), w1l, b1l))
        part = torch.nn.functional.linear(h, w2l)
        dist.reduce_scatter_tensor(rs_out, part)
        return rs_out
    out["mlp_fused_ms"] = timed(mlp.forward)
    out["mlp_nccl_torch_ms"] = timed(mlp_baseline)
    comm.check("tp worker")
    # roofline of the fused kernels: max(FLOPs / measured GEMM peak, NVLink bytes / 770 GB/s)
    flops = 2.0 * M * K * nl
    nv_bytes = (world - 1) / world * M * K * 2
    out["col_roofline_ms"] = max(flops / 1404.3e12, nv_bytes / 770e9) * 1e3
    flops2 = 2.0 * M * kl * N2
    nv2 = (world - 1) / world * M * N2 * 2
    out["row_roofline_ms"] = max(flops2 / 1404.3e12, nv2 / 770e9) * 1e3
    if rank == 0:
        print("TPRESULT " + json.dumps(out), flush=True)
    comm.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
