"""LayerNorm, embedding + LayerNorm, masked softmax, composed and fused attention vs PyTorch fp32."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
F = torch.nn.functional


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("c", [768, 1280, 64])
def test_layernorm(dtype, c):
    from fastdeploy_b200.ops import transformer as T
    torch.manual_seed(0)
    x = torch.randn(300, c, device="cuda").to(dtype)
    g = torch.rand(c, device="cuda") + 0.5
    b = torch.randn(c, device="cuda")
    y = torch.empty_like(x)
    T.layernorm(x, y, g, b, rows=300, c=c, eps=1e-5).launch()
    ref = F.layer_norm(x.float(), [c], g, b, 1e-5)
    assert (y.float() - ref).abs().max().item() < (3e-2 if dtype == torch.bfloat16 else 5e-3)


def test_embed_layernorm():
    from fastdeploy_b200.ops import transformer as T
    torch.manual_seed(1)
    bsz, seq, c = 3, 20, 768
    word = (torch.randn(1000, c, device="cuda") * 0.1).half()
    pos = (torch.randn(64, c, device="cuda") * 0.1).half()
    typ = (torch.randn(4, c, device="cuda") * 0.1).half()
    ids = torch.randint(0, 1000, (bsz * seq,), device="cuda")
    tids = torch.randint(0, 4, (bsz * seq,), device="cuda")
    g = torch.rand(c, device="cuda") + 0.5
    b = torch.randn(c, device="cuda")
    y = torch.empty(bsz * seq, c, device="cuda", dtype=torch.float16)
    T.embed_layernorm([ids, None, tids], [word, pos, typ], y, g, b, rows=bsz * seq, c=c, seq=seq).launch()
    p = torch.arange(bsz * seq, device="cuda") % seq
    ref = F.layer_norm(word[ids].float() + pos[p].float() + typ[tids].float(), [c], g, b, 1e-5)
    assert (y.float() - ref).abs().max().item() < 1e-2


@pytest.mark.parametrize("cfg", [(2, 4, 128, 64, True), (3, 2, 50, 64, True), (2, 16, 257, 80, False),
                                 (1, 12, 512, 64, True)])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("fused", [True, False])
def test_attention(cfg, dtype, fused):
    from fastdeploy_b200.ops.transformer import Attention
    b, h, s, d, use_mask = cfg
    torch.manual_seed(2)
    qkv = (torch.randn(b, s, 3 * h * d, device="cuda") * 0.5).to(dtype)     # fused QKV buffer
    q, k, v = qkv[..., :h * d], qkv[..., h * d:2 * h * d], qkv[..., 2 * h * d:]
    mask = None
    if use_mask:
        lens = torch.randint(s // 2, s + 1, (b,))
        mask = torch.zeros(b, 1, 1, s, device="cuda")
        for i in range(b):
            mask[i, ..., lens[i]:] = -1e4
    out = torch.zeros(b, s, h * d, device="cuda", dtype=dtype)
    att = Attention(q, k, v, out, heads=h, scale=1 / math.sqrt(d), mask=mask, fused=fused)
    assert att.fused == fused
    att.launch()
    att.status.check()

    def split(t):
        return t.float().reshape(b, s, h, d).permute(0, 2, 1, 3)
    sc = split(q) @ split(k).transpose(-1, -2) / math.sqrt(d)
    if mask is not None:
        sc = sc + mask
    ref = (torch.softmax(sc, -1) @ split(v)).permute(0, 2, 1, 3).reshape(b, s, h * d)
    tol = 3e-2 if dtype == torch.bfloat16 else 6e-3
    assert (out.float() - ref).abs().max().item() < tol
