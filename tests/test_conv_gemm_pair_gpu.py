"""CTA-pair (cta_group::2) form of the implicit-GEMM kernel against fp32 references: element-wise
``atol + rtol * |ref|`` bounds with TF32 off, and integer-valued cases that must match exactly
(every product and partial sum is representable, so a dropped K tail, a wrong weight half or a swapped
tile shows up as a hard mismatch instead of hiding under a norm)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _no_tf32():
    old = (torch.backends.cudnn.allow_tf32, torch.backends.cuda.matmul.allow_tf32)
    torch.backends.cudnn.allow_tf32 = False
    torch.backends.cuda.matmul.allow_tf32 = False
    yield
    torch.backends.cudnn.allow_tf32, torch.backends.cuda.matmul.allow_tf32 = old


def _close(y, ref, atol, rtol):
    err = (y.float() - ref).abs()
    bound = atol + rtol * ref.abs()
    bad = err > bound
    assert not bool(bad.any()), f"{int(bad.sum())} elements out of bound, worst {float((err - bound).max())}"


def _ints(shape, lo, hi, dtype):
    return torch.randint(lo, hi + 1, shape, device="cuda").to(dtype)


@pytest.mark.parametrize("m,k,n", [(256, 64, 128), (300, 64, 192), (1000, 200, 264), (4096, 1280, 768), (129, 72, 64)])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_pair_gemm_exact_on_integers(m, k, n, dtype):
    from fastdeploy_b200.ops.conv_gemm import ConvGemm, pack_linear_weight
    torch.manual_seed(0)
    x = _ints((m, k), -2, 2, dtype)
    w = _ints((n, k), -1, 1, dtype)
    b = _ints((n,), -3, 3, torch.float32)
    y = torch.full((m, (n + 7) // 8 * 8), 7.0, device="cuda")
    op = ConvGemm(x, pack_linear_weight(w, dtype), y, in_shape=(1, 1, m, k), out_hw=(1, m), cout=n, bias=b,
                  y_ld=y.stride(0), pair_mode=1)
    assert op.info()["variant"] == 3
    op.launch()
    op.status.check("pair gemm")
    ref = x.float() @ w.float().t() + b
    assert torch.equal(y[:, :n], ref)
    assert bool((y[:, n:] == 7.0).all())          # padding columns untouched


@pytest.mark.parametrize("m,k,n,act", [(512, 256, 256, "gelu"), (777, 768, 192, None), (2048, 512, 640, "silu")])
def test_pair_gemm_random_16bit_output(m, k, n, act):
    from fastdeploy_b200.ops.conv_gemm import linear
    torch.manual_seed(1)
    x = (torch.randn(m, k, device="cuda") * 0.5).half()
    w = (torch.randn(n, k, device="cuda") * 0.05).half()
    b = torch.randn(n, device="cuda")
    res = (torch.randn(m, n, device="cuda") * 0.5).half()
    y = linear(x, w, b, act=act, residual=res, res_mode=2, pair_mode=1)
    z = x.float() @ w.float().t() + b
    if act == "gelu":
        z = torch.nn.functional.gelu(z)
    elif act == "silu":
        z = torch.nn.functional.silu(z)
    _close(y, z + res.float(), atol=6e-3, rtol=4e-3)
    same = linear(x, w, b, act=act, residual=res, res_mode=2, pair_mode=0)
    _close(y, same.float(), atol=4e-3, rtol=2e-3)


@pytest.mark.parametrize("cfg", [
    # n, h, w, cin, cout, k, stride, pad
    (3, 20, 20, 64, 128, 3, 1, 1),
    (2, 40, 40, 96, 192, 3, 2, 1),
    (5, 13, 17, 72, 64, 1, 1, 0),
    (1, 33, 47, 32, 80, 3, 1, 1),
])
def test_pair_conv_exact_on_integers(cfg):
    from fastdeploy_b200.ops.conv_gemm import ConvGemm, pack_conv_weight
    n, h, w_, cin, cout, k, s, p = cfg
    torch.manual_seed(2)
    x = _ints((n, h, w_, cin), -1, 1, torch.float16)
    w = _ints((cout, cin, k, k), -1, 1, torch.float16)
    b = _ints((cout,), -2, 2, torch.float32)
    ho, wo = (h + 2 * p - k) // s + 1, (w_ + 2 * p - k) // s + 1
    ybuf = torch.zeros(n, ho, wo, cout + 16, device="cuda")
    op = ConvGemm(x, pack_conv_weight(w, torch.float16), ybuf[..., 8:], in_shape=(n, h, w_, cin), out_hw=(ho, wo),
                  cout=cout, kernel=(k, k), stride=s, pad=(p, p), bias=b, y_ld=cout + 16, halo_mode=0, pair_mode=1)
    assert op.info()["variant"] == 3
    op.launch()
    op.status.check("pair conv")
    ref = _int_conv_ref(x, w, b, s, p)
    assert torch.equal(ybuf[..., 8:8 + cout], ref)
    assert float(ybuf[..., :8].abs().max()) == 0 and float(ybuf[..., 8 + cout:].abs().max()) == 0


def _int_conv_ref(x, w, b, s, p):
    """Exact integer result: the library convolution may pick a transform-domain algorithm that is off by
    rounding noise, so its output is rounded to the integers the true result consists of."""
    ref = torch.nn.functional.conv2d(x.float().permute(0, 3, 1, 2), w.float(), b, stride=s, padding=p).permute(0, 2, 3, 1)
    assert float((ref - ref.round()).abs().max()) < 1e-3
    return ref.round()


@pytest.mark.parametrize("cfg", [
    # n, h, w, cin, cout   (3x3, stride 1, pad 1: the halo kernel on CTA pairs)
    (3, 20, 20, 96, 96),        # weights resident per CTA half
    (2, 40, 40, 192, 192),      # weights streamed
    (5, 16, 24, 64, 128),
    (1, 33, 47, 40, 80),        # ragged tiles, odd tile count, channel tail
    (3, 16, 16, 384, 384),      # two column tiles
])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_pair_halo_conv_exact_on_integers(cfg, dtype):
    from fastdeploy_b200.ops.conv_gemm import ConvGemm, pack_conv_weight
    n, h, w_, cin, cout = cfg
    torch.manual_seed(5)
    x = _ints((n, h, w_, cin), -1, 1, dtype)
    w = _ints((cout, cin, 3, 3), -1, 1, dtype)
    b = _ints((cout,), -2, 2, torch.float32)
    y = torch.zeros(n, h, w_, cout, device="cuda", dtype=dtype)
    op = ConvGemm(x, pack_conv_weight(w, dtype), y, in_shape=(n, h, w_, cin), out_hw=(h, w_), cout=cout,
                  kernel=(3, 3), stride=1, pad=(1, 1), bias=b, halo_mode=1, pair_mode=1)
    assert op.info()["variant"] in (4, 5)
    op.launch()
    op.status.check("pair halo conv")
    ref = _int_conv_ref(x, w, b, 1, 1)
    if dtype == torch.bfloat16:                 # sums beyond 256 are not representable in bf16
        ref = ref.to(torch.bfloat16).float()
    assert torch.equal(y.float(), ref)


def test_pair_halo_conv_random_residual():
    from fastdeploy_b200.ops.conv_gemm import ConvGemm, pack_conv_weight
    torch.manual_seed(6)
    n, h, w_, cin, cout = 4, 40, 40, 96, 96
    x = (torch.randn(n, h, w_, cin, device="cuda") * 0.5).half()
    w = (torch.randn(cout, cin, 3, 3, device="cuda") * 0.03).half()
    b = torch.randn(cout, device="cuda") * 0.1
    res = (torch.randn(n, h, w_, cout, device="cuda") * 0.5).half()
    y = torch.zeros(n, h, w_, cout, device="cuda", dtype=torch.float16)
    op = ConvGemm(x, pack_conv_weight(w, torch.float16), y, in_shape=(n, h, w_, cin), out_hw=(h, w_), cout=cout,
                  kernel=(3, 3), stride=1, pad=(1, 1), bias=b, residual=res, res_mode=2, act="silu", halo_mode=1,
                  pair_mode=1)
    assert op.info()["variant"] == 5
    for _ in range(3):                          # resident weights survive across launches
        op.launch()
    op.status.check("pair halo conv")
    z = torch.nn.functional.conv2d(x.float().permute(0, 3, 1, 2), w.float(), b, padding=1).permute(0, 2, 3, 1)
    _close(y, torch.nn.functional.silu(z) + res.float(), atol=8e-3, rtol=4e-3)


def test_pair_conv_fp16_out_residual_slices():
    from fastdeploy_b200.ops.conv_gemm import ConvGemm, pack_conv_weight
    torch.manual_seed(3)
    n, h, w_, cin, cout = 3, 20, 20, 128, 192
    xbuf = (torch.randn(n, h, w_, 256, device="cuda") * 0.5).half()
    x = xbuf[..., 128:]
    ybuf = torch.zeros(n, h, w_, 384, device="cuda", dtype=torch.float16)
    res = (torch.randn(n, h, w_, cout, device="cuda") * 0.5).half()
    w = (torch.randn(cout, cin, 3, 3, device="cuda") * 0.03).half()
    b = torch.randn(cout, device="cuda") * 0.1
    op = ConvGemm(x, pack_conv_weight(w, torch.float16), ybuf[..., 192:], in_shape=(n, h, w_, cin), out_hw=(h, w_),
                  cout=cout, kernel=(3, 3), stride=1, pad=(1, 1), bias=b, residual=res, res_mode=2, act="silu",
                  x_ld=256, y_ld=384, halo_mode=0, pair_mode=1)
    op.launch()
    op.status.check("pair conv")
    z = torch.nn.functional.conv2d(x.float().permute(0, 3, 1, 2), w.float(), b, padding=1).permute(0, 2, 3, 1)
    ref = torch.nn.functional.silu(z) + res.float()
    _close(ybuf[..., 192:], ref, atol=8e-3, rtol=4e-3)
    assert float(ybuf[..., :192].abs().max()) == 0
