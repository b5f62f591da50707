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


@pytest.mark.parametrize("cfg", [(4, 4, 128, 64), (3, 12, 384, 64), (2, 16, 257, 80)])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_attention_with_per_item_lengths(cfg, dtype):
    """Padded batch + a device tensor of lengths: real rows match per-item attention over the item's own tokens,
    rows past an item's length are left as they were; the lengths are re-read at every launch."""
    from fastdeploy_b200.ops.transformer import Attention
    b, h, s, d = cfg
    torch.manual_seed(5)
    qkv = (torch.randn(b, s, 3 * h * d, device="cuda") * 0.5).to(dtype)
    q, k, v = qkv[..., :h * d], qkv[..., h * d:2 * h * d], qkv[..., 2 * h * d:]
    lens = torch.zeros(b, dtype=torch.int32, device="cuda")
    out = torch.zeros(b, s, h * d, device="cuda", dtype=dtype)
    att = Attention(q, k, v, out, heads=h, scale=1 / math.sqrt(d), seq_lens=lens)
    tol = 3e-2 if dtype == torch.bfloat16 else 6e-3
    for trial in range(2):
        host = [s, 1, 17, s // 2 + 3][:b] if trial == 0 else [5, s, s - 1, min(130, s)][:b]
        lens.copy_(torch.tensor(host, dtype=torch.int32))
        out.fill_(7.0)
        att.launch()
        att.status.check()
        for i, n in enumerate(host):
            def split(t):
                return t[i, :n].float().reshape(n, h, d).permute(1, 0, 2)
            sc = split(q) @ split(k).transpose(-1, -2) / math.sqrt(d)
            ref = (torch.softmax(sc, -1) @ split(v)).permute(1, 0, 2).reshape(n, h * d)
            assert (out[i, :n].float() - ref).abs().max().item() < tol, (trial, i, n)
            assert (out[i, n:] == 7.0).all()


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_packed_attention_matches_per_sequence_attention(dtype):
    """Padding-free batch: sequences back to back at 8-row aligned starts, one planned op for two compositions."""
    from fastdeploy_b200.ops.transformer import PackedAttention, pack_offsets
    h, d, max_len, max_seqs, rows = 12, 64, 512, 6, 1536
    torch.manual_seed(6)
    qkv = (torch.randn(rows, 3 * h * d, device="cuda") * 0.5).to(dtype)
    q, k, v = qkv[:, :h * d], qkv[:, h * d:2 * h * d], qkv[:, 2 * h * d:]
    out = torch.zeros(rows, h * d, device="cuda", dtype=dtype)
    start = torch.zeros(max_seqs, dtype=torch.int32, device="cuda")
    lens = torch.zeros(max_seqs, dtype=torch.int32, device="cuda")
    att = PackedAttention(q, k, v, out, heads=h, scale=1 / math.sqrt(d), max_len=max_len, seq_start=start, seq_len=lens)
    tol = 3e-2 if dtype == torch.bfloat16 else 6e-3
    for host in ([512, 3, 100, 257, 64, 300], [130, 511, 9]):
        starts, total = pack_offsets(host)
        assert total <= rows and all(x % 8 == 0 for x in starts)
        pad = max_seqs - len(host)
        start.copy_(torch.tensor(starts + [0] * pad, dtype=torch.int32))
        lens.copy_(torch.tensor(list(host) + [0] * pad, dtype=torch.int32))
        out.fill_(7.0)
        att.launch()
        att.status.check()
        covered = torch.zeros(rows, dtype=torch.bool, device="cuda")
        for st, n in zip(starts, host):
            def split(t):
                return t[st:st + n].float().reshape(n, h, d).permute(1, 0, 2)
            sc = split(q) @ split(k).transpose(-1, -2) / math.sqrt(d)
            ref = (torch.softmax(sc, -1) @ split(v)).permute(1, 0, 2).reshape(n, h * d)
            assert (out[st:st + n].float() - ref).abs().max().item() < tol, (st, n)
            covered[st:st + n] = True
        assert (out[~covered] == 7.0).all()


def test_packed_attention_reports_a_misaligned_start():
    """A start that is not a multiple of 8 rows is refused by the kernel (status word), not loaded."""
    from fastdeploy_b200.ops.transformer import PackedAttention
    h, d, rows = 4, 64, 256
    qkv = torch.zeros(rows, 3 * h * d, device="cuda", dtype=torch.float16)
    out = torch.zeros(rows, h * d, device="cuda", dtype=torch.float16)
    start = torch.tensor([0, 12], dtype=torch.int32, device="cuda")
    lens = torch.tensor([10, 20], dtype=torch.int32, device="cuda")
    att = PackedAttention(qkv[:, :h * d], qkv[:, h * d:2 * h * d], qkv[:, 2 * h * d:], out, heads=h, scale=0.125,
                          max_len=128, seq_start=start, seq_len=lens)
    att.launch()
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError):
        att.status.check()


@pytest.mark.parametrize("kind", ["prefix", "holes", "soft", "all_masked_item"])
def test_attention_mask_kinds(kind):
    """A key-padding mask (zeros, then <= -1000) runs from its key count; any other mask is added to the scores.
    Both give softmax(q k^T * scale + mask) v for every query row, padded ones included."""
    from fastdeploy_b200.ops.transformer import Attention
    b, h, s, d = 3, 4, 200, 64
    torch.manual_seed(9)
    qkv = (torch.randn(b, s, 3 * h * d, device="cuda") * 0.5).half()
    q, k, v = qkv[..., :h * d], qkv[..., h * d:2 * h * d], qkv[..., 2 * h * d:]
    mask = torch.zeros(b, 1, 1, s, device="cuda")
    mask[0, ..., 150:] = -1e4
    mask[1, ..., 7:] = -1e4
    if kind == "holes":
        mask[2, ..., 50:60] = -1e4                  # not a prefix: the general path
    elif kind == "soft":
        mask[2, ..., 100:] = -3.0                   # finite bias: must be added, not dropped
    elif kind == "all_masked_item":
        mask[2] = -1e4                              # no key left: uniform weights, as the formula gives
    out = torch.zeros(b, s, h * d, device="cuda", dtype=torch.float16)
    att = Attention(q, k, v, out, heads=h, scale=1 / math.sqrt(d), mask=mask)
    assert att.fused
    for _ in range(2):                              # the key counts are recomputed at every launch
        att.launch()
    att.status.check()

    def split(t):
        return t.float().reshape(b, s, h, d).permute(0, 2, 1, 3)
    sc = split(q) @ split(k).transpose(-1, -2) / math.sqrt(d) + mask
    ref = (torch.softmax(sc, -1) @ split(v)).permute(0, 2, 1, 3).reshape(b, s, h * d)
    assert (out.float() - ref).abs().max().item() < 6e-3
