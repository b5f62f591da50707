"""Tensor-parallel ViT against the fp32 PyTorch forward of the same weights: one rank on one GPU, and two
ranks (child processes under torchrun) where two GPUs are present."""
import json
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ARGS = ["-m", "fastdeploy_b200.parallel.bench_vit", "--size", "test", "--batch", "8", "--image", "28", "--classes", "16",
        "--steps", "0", "--check"]


def _result(p):
    assert p.returncode == 0, p.stdout[-3000:] + p.stderr[-3000:]
    line = [l for l in p.stdout.splitlines() if l.startswith("TPVIT ")][-1]
    return json.loads(line[len("TPVIT "):])


def test_vit_one_rank_matches_fp32_reference():
    p = subprocess.run([sys.executable] + ARGS, capture_output=True, text=True, timeout=600, cwd=ROOT)
    r = _result(p)
    assert r["max_abs_err"] < 0.03 * r["ref_max_prob"], r
    assert r["top1_agree"] >= 0.75, r


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_vit_two_ranks_match_fp32_reference():
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", "29543"] + ARGS
    r = _result(subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=ROOT))
    assert r["world"] == 2
    assert r["max_abs_err"] < 0.03 * r["ref_max_prob"], r
    assert r["top1_agree"] >= 0.75, r


def test_vit_fp8_one_rank_close_to_fp32_reference():
    """e4m3 linears with calibrated static activation scales: the class probabilities stay close to the fp32
    forward and the arg-max class agrees on most images (random weights give nearly flat distributions, so the
    agreement bound is loose and the error bound carries the check)."""
    p = subprocess.run([sys.executable] + ARGS + ["--dtype", "fp8"], capture_output=True, text=True, timeout=600, cwd=ROOT)
    r = _result(p)
    assert r["dtype"] == "fp8"
    assert r["max_abs_err"] < 0.12 * r["ref_max_prob"], r
    assert r["top1_agree"] >= 0.6, r


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_vit_fp8_two_ranks_close_to_fp32_reference():
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", "29544"] + ARGS + ["--dtype", "fp8"]
    r = _result(subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=ROOT))
    assert r["world"] == 2 and r["dtype"] == "fp8"
    assert r["max_abs_err"] < 0.12 * r["ref_max_prob"], r
    assert r["top1_agree"] >= 0.6, r


@pytest.mark.parametrize("world", [4, 8])
@pytest.mark.parametrize("dtype", ["bf16", "fp8"])
def test_vit_four_and_eight_ranks_match_fp32_reference(world, dtype):
    """The fused GEMM + collective kernels with 4 and 8 ranks (pull reduce-scatter from 3 / 7 peers, copier
    CTAs gathering from 3 / 7 peers); skipped where the box has fewer GPUs."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    args = list(ARGS)
    args[args.index("--batch") + 1] = "24"          # 24 images x 5 tokens: every rank owns real rows at 8 ranks too
    args[args.index("--size") + 1] = "test8"        # 8 heads, so the heads divide over 8 ranks
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr",
           "127.0.0.1", "--master-port", str(29560 + world)] + args + ["--dtype", dtype]
    r = _result(subprocess.run(cmd, capture_output=True, text=True, timeout=900, env=env, cwd=ROOT))
    assert r["world"] == world
    tol = 0.12 if dtype == "fp8" else 0.03
    assert r["max_abs_err"] < tol * r["ref_max_prob"], r
    assert r["top1_agree"] >= (0.6 if dtype == "fp8" else 0.75), r


def test_vit_eight_head_test_size_on_one_rank():
    """The size used by the 4- and 8-rank tests, checked where one GPU is enough."""
    args = list(ARGS)
    args[args.index("--size") + 1] = "test8"
    r = _result(subprocess.run([sys.executable] + args, capture_output=True, text=True, timeout=600, cwd=ROOT))
    assert r["max_abs_err"] < 0.03 * r["ref_max_prob"], r
