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
