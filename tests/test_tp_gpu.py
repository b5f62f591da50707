"""Tensor-parallel kernels on 2+ GPUs (child processes under torchrun) and the bounded peer wait."""
import json
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_peer_wait_times_out_with_status_not_a_hang():
    """A barrier whose second participant never arrives (its slot is in this rank's own heap and
    nothing bumps it) must give up after its clock budget and report through the status word."""
    import ctypes
    from fastdeploy_b200.ops.base import StatusWord, current_stream_ptr
    from fastdeploy_b200.parallel.comm import _lib
    lib = _lib()
    base = lib.fdb_comm_alloc(4096)
    assert base
    st = StatusWord(torch.device("cuda"))
    flags = (ctypes.c_void_p * 8)()
    flags[0] = base
    flags[1] = base + 1024          # stands in for a peer that never signals
    assert lib.fdb_comm_barrier(flags, 2, 0, 1, st.ptr, ctypes.c_void_p(current_stream_ptr())) == 0
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match="peer signal wait timed out"):
        st.check("barrier")
    # the context is still usable
    assert float(torch.ones(4, device="cuda").sum()) == 4.0
    lib.fdb_comm_free(base)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_tp_worker_two_ranks():
    n = 2
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
           "--master-addr", "127.0.0.1", "--master-port", "29533", os.path.join(ROOT, "tests", "tp_worker.py")]
    p = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)
    assert p.returncode == 0, p.stdout[-3000:] + p.stderr[-3000:]
    line = [l for l in p.stdout.splitlines() if l.startswith("TPRESULT ")][-1]
    r = json.loads(line[len("TPRESULT "):])
    assert r["allreduce_err"] < 0.1 and r["reducescatter_err"] < 0.1 and r["allgather_err"] == 0.0
    assert r["col_err"] < 2e-2 and r["row_err"] < 2e-2 and r["mlp_err"] < 2e-2, r


@pytest.mark.parametrize("world", [1, 2, 8])
def test_slot_reduce_with_residual_and_layernorm_matches_fp32(world):
    """The kernel behind every row-parallel GEMM of the tensor-parallel ViT, fed by hand on one GPU: partial blocks
    of `world` ranks already sit in the slots and the arrival counters already hold the target."""
    import ctypes
    from fastdeploy_b200.ops.base import StatusWord, current_stream_ptr, dtype_code
    from fastdeploy_b200.parallel.comm import _lib
    torch.manual_seed(0)
    rows, cols = 300, 1280
    dev = "cuda"
    slots = (torch.randn(world, rows, cols, device=dev) * 0.3).bfloat16()
    x = torch.randn(rows, cols, device=dev).bfloat16()
    bias = torch.randn(cols, device=dev)
    gamma, beta = torch.rand(cols, device=dev) + 0.5, torch.randn(cols, device=dev)
    y = torch.zeros(rows, cols, device=dev, dtype=torch.bfloat16)
    counters = torch.full(((rows + 127) // 128,), 7, dtype=torch.int32, device=dev)
    x_ref = (x.float() + bias + slots.float().sum(0)).bfloat16()
    y_ref = torch.nn.functional.layer_norm(x_ref.float(), (cols,), gamma, beta, 1e-6)
    st = StatusWord(torch.device(dev))
    P = ctypes.c_void_p
    rc = _lib().fdb_comm_slot_reduce_ln(P(slots.data_ptr()), P(counters.data_ptr()), 7, P(x.data_ptr()), P(bias.data_ptr()),
                                        rows, cols, world, dtype_code(torch.bfloat16), st.ptr, P(gamma.data_ptr()),
                                        P(beta.data_ptr()), 1e-6, P(y.data_ptr()), cols, P(current_stream_ptr()), 0, 1.0)
    assert rc == 0
    torch.cuda.synchronize()
    st.check("slot_reduce_ln")
    assert (x.float() - x_ref.float()).abs().max().item() <= 0.0625       # one bf16 step at these magnitudes
    assert (y.float() - y_ref).abs().max().item() < 0.1                   # bf16 output, values up to about 10
    assert (y.float() - y_ref).abs().mean().item() < 5e-3
