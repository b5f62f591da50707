"""The checked kernel library (-DFDB_BOUNDS_CHECK) counts data-dependent indices that the release build clamps."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = r"""
import torch
from fastdeploy_b200 import _native
from fastdeploy_b200.ops import generic as G, transformer as T
assert _native.kernels().fdb_bounds_checked() == 1
assert _native.bounds_report()[0] == 0
table = torch.arange(40, device="cuda", dtype=torch.float32).reshape(10, 4)
index = torch.tensor([0, 9, 12, -1, -30], device="cuda")           # 12 and -30 are out of range, -1 is row 9
out = torch.zeros(5, 4, device="cuda")
G.gather_rows(table, index, out).launch()
torch.cuda.synchronize()
assert out[:, 0].tolist() == [0.0, 36.0, 36.0, 36.0, 0.0]          # clamped, never read outside the table
n, text = _native.bounds_report()
assert n == 2 and "unit=generic_ops" in text and "site=1" in text and "extent=10" in text, text
assert _native.bounds_report()[0] == 0                              # the report reset the record
c, rows = 64, 6
word = torch.randn(50, c, device="cuda").half()
pos = torch.randn(8, c, device="cuda").half()
ids = torch.tensor([1, 49, 50, 7, 1000, 3], device="cuda")
y = torch.zeros(rows, c, device="cuda", dtype=torch.float16)
g, b = torch.ones(c, device="cuda"), torch.zeros(c, device="cuda")
T.embed_layernorm([ids, None], [word, pos], y, g, b, rows=rows, c=c, seq=6).launch()
torch.cuda.synchronize()
ref = torch.nn.functional.layer_norm(word[ids.clamp(0, 49)].float() + pos[torch.arange(6, device="cuda")].float(), [c])
assert (y.float() - ref).abs().max().item() < 1e-2
n, text = _native.bounds_report()
assert n == 2 and "unit=transformer_ops" in text and "site=2" in text, text
print("checked build ok")
"""


def test_checked_kernel_library_reports_clamped_indices():
    from fastdeploy_b200._native import build as B
    lib = B.variant_lib("boundscheck")
    if not os.path.exists(lib):
        pytest.skip("build/boundscheck is not built: python -m fastdeploy_b200._native.build --mode boundscheck")
    env = dict(os.environ, FDX_NATIVE_VARIANT="boundscheck")
    run = subprocess.run([sys.executable, "-c", CHILD], cwd=ROOT, env=env, stdout=subprocess.PIPE,
                         stderr=subprocess.STDOUT, text=True, timeout=600)
    assert run.returncode == 0 and "checked build ok" in run.stdout, run.stdout[-4000:]


def test_release_library_clamps_token_ids_outside_the_table():
    import torch
    from fastdeploy_b200 import _native
    from fastdeploy_b200.ops import transformer as T
    c = 64
    word = torch.randn(50, c, device="cuda").half()
    ids = torch.tensor([49, 50, -4, 7], device="cuda")
    y = torch.zeros(4, c, device="cuda", dtype=torch.float16)
    T.embed_layernorm([ids], [word], y, torch.ones(c, device="cuda"), torch.zeros(c, device="cuda"), rows=4, c=c,
                      seq=4).launch()
    torch.cuda.synchronize()
    ref = torch.nn.functional.layer_norm(word[ids.clamp(0, 49)].float(), [c])
    assert (y.float() - ref).abs().max().item() < 1e-2
    assert _native.bounds_report()[1] == "not a checked build"
