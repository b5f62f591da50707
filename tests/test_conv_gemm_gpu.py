"""tcgen05 implicit-GEMM conv / GEMM against a plain PyTorch fp32 reference."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref_conv(x_nhwc, w, b, stride, pad, act, residual=None, res_mode=0):
    x = x_nhwc.float().permute(0, 3, 1, 2)
    y = torch.nn.functional.conv2d(x, w.float(), b.float() if b is not None else None, stride=stride, padding=pad)
    y = y.permute(0, 2, 3, 1)
    if residual is not None and res_mode == 1:
        y = y + residual.float()
    if act == "silu":
        y = torch.nn.functional.silu(y)
    elif act == "relu":
        y = torch.relu(y)
    elif act == "gelu":
        y = torch.nn.functional.gelu(y)
    elif act == "hard_swish":
        y = torch.nn.functional.hardswish(y)
    if residual is not None and res_mode == 2:
        y = y + residual.float()
    return y


def _check(y, ref, tol=2e-2):
    err = (y.float() - ref).abs().max().item()
    scale = ref.abs().max().item() + 1e-6
    assert err / scale < tol, f"max abs err {err} vs scale {scale}"


@pytest.mark.parametrize("m,k,n", [(128, 64, 32), (256, 128, 64), (300, 192, 80), (1000, 768, 768), (4096, 1024, 2304),
                                   (257, 1280, 5120)])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_linear(m, k, n, dtype):
    from fastdeploy_b200.ops.conv_gemm import linear
    torch.manual_seed(0)
    x = (torch.randn(m, k, device="cuda") * 0.5).to(dtype)
    w = (torch.randn(n, k, device="cuda") * 0.05).to(dtype)
    b = torch.randn(n, device="cuda")
    y = linear(x, w, b, act="gelu")
    ref = torch.nn.functional.gelu(x.float() @ w.float().t() + b)
    _check(y, ref)


@pytest.mark.parametrize("block_n", [32, 48, 64, 80, 96, 128, 160, 192, 256])
def test_linear_block_n(block_n):
    from fastdeploy_b200.ops.conv_gemm import linear
    torch.manual_seed(1)
    x = (torch.randn(520, 256, device="cuda") * 0.5).half()
    w = (torch.randn(264, 256, device="cuda") * 0.05).half()
    y = linear(x, w, None, block_n=block_n, out_dtype=torch.float32)
    _check(y, x.float() @ w.float().t())


@pytest.mark.parametrize("cfg", [
    # n, h, w, cin, cout, k, stride, pad, act
    (2, 16, 16, 64, 64, 1, 1, 0, None),
    (2, 16, 16, 64, 64, 3, 1, 1, "silu"),
    (3, 20, 20, 128, 96, 3, 1, 1, "relu"),
    (2, 40, 40, 96, 192, 3, 1, 1, "silu"),
    (1, 33, 47, 32, 40, 3, 1, 1, "hard_swish"),
    (2, 24, 24, 16, 24, 5, 1, 2, None),
])
def test_conv_stride1(cfg):
    from fastdeploy_b200.ops.conv_gemm import conv2d_nhwc
    n, h, w_, cin, cout, k, s, p, act = cfg
    torch.manual_seed(2)
    x = (torch.randn(n, h, w_, cin, device="cuda") * 0.5).half()
    w = (torch.randn(cout, cin, k, k, device="cuda") * (1.0 / (cin * k * k) ** 0.5)).half()
    b = torch.randn(cout, device="cuda") * 0.1
    y = conv2d_nhwc(x, w, b, stride=s, pad=p, act=act)
    _check(y, _ref_conv(x, w, b, s, p, act))


@pytest.mark.parametrize("cfg", [
    (2, 16, 16, 64, 64, 3, 2, 1, "silu"),
    (2, 40, 40, 64, 128, 3, 2, 1, "silu"),
    (1, 33, 47, 32, 48, 3, 2, 1, None),
    (2, 32, 32, 64, 64, 1, 2, 0, None),
])
def test_conv_stride2(cfg):
    from fastdeploy_b200.ops.conv_gemm import conv2d_nhwc
    n, h, w_, cin, cout, k, s, p, act = cfg
    torch.manual_seed(3)
    x = (torch.randn(n, h, w_, cin, device="cuda") * 0.5).half()
    w = (torch.randn(cout, cin, k, k, device="cuda") * (1.0 / (cin * k * k) ** 0.5)).half()
    b = torch.randn(cout, device="cuda") * 0.1
    y = conv2d_nhwc(x, w, b, stride=s, pad=p, act=act)
    _check(y, _ref_conv(x, w, b, s, p, act))


@pytest.mark.parametrize("res_mode", [1, 2])
def test_conv_residual_and_concat_slice(res_mode):
    """Residual epilogue, and writing into / reading from a channel slice of a wider buffer."""
    from fastdeploy_b200.ops.conv_gemm import ConvGemm, pack_conv_weight
    torch.manual_seed(4)
    n, h, w_, cin, cout = 2, 20, 20, 64, 64
    xbuf = (torch.randn(n, h, w_, 128, device="cuda") * 0.5).half()
    x = xbuf[..., 64:]                      # input = upper channel half of a concat buffer
    ybuf = torch.zeros(n, h, w_, 192, device="cuda", dtype=torch.float16)
    res = (torch.randn(n, h, w_, cout, device="cuda") * 0.5).half()
    w = (torch.randn(cout, cin, 3, 3, device="cuda") * 0.04).half()
    b = torch.randn(cout, device="cuda") * 0.1
    op = ConvGemm(x, pack_conv_weight(w, torch.float16), ybuf[..., 128:], in_shape=(n, h, w_, cin), out_hw=(h, w_),
                  cout=cout, kernel=(3, 3), stride=1, pad=(1, 1), bias=b, residual=res, res_mode=res_mode,
                  act="silu", x_ld=128, y_ld=192)
    op.launch()
    op.status.check()
    ref = _ref_conv(x.contiguous(), w, b, 1, 1, "silu", res, res_mode)
    _check(ybuf[..., 128:], ref)
    assert float(ybuf[..., :128].abs().max()) == 0.0


def test_conv_image_strides_and_fp32_out():
    """Per-image strides: levels of a detection head land in one [N, anchors, C] buffer."""
    from fastdeploy_b200.ops.conv_gemm import ConvGemm, pack_conv_weight
    torch.manual_seed(5)
    n, h, w_, cin, cout = 3, 10, 10, 64, 68
    x = (torch.randn(n, h, w_, cin, device="cuda") * 0.5).half()
    w = (torch.randn(cout, cin, 3, 3, device="cuda") * 0.04).half()
    b = torch.randn(cout, device="cuda") * 0.1
    total = 250
    ybuf = torch.zeros(n, total, cout, device="cuda", dtype=torch.float32)
    op = ConvGemm(x, pack_conv_weight(w, torch.float16), ybuf[:, 150:], in_shape=(n, h, w_, cin), out_hw=(h, w_),
                  cout=cout, kernel=(3, 3), stride=1, pad=(1, 1), bias=b, act="sigmoid", y_n_stride=total * cout)
    op.launch()
    op.status.check()
    ref = torch.sigmoid(_ref_conv(x, w, b, 1, 1, None)).reshape(n, h * w_, cout)
    _check(ybuf[:, 150:], ref, tol=5e-3)
    assert float(ybuf[:, :150].abs().max()) == 0.0


@pytest.mark.parametrize("act", ["relu", "silu", "hard_swish", "sigmoid", "gelu", "relu6", "tanh", None])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_linear_activations(act, dtype):
    from fastdeploy_b200.ops.conv_gemm import linear
    torch.manual_seed(6)
    x = (torch.randn(300, 128, device="cuda")).to(dtype)
    w = (torch.randn(96, 128, device="cuda") * 0.1).to(dtype)
    b = torch.randn(96, device="cuda")
    y = linear(x, w, b, act=act)
    z = x.float() @ w.float().t() + b
    F = torch.nn.functional
    ref = {None: lambda t: t, "relu": torch.relu, "silu": F.silu, "hard_swish": F.hardswish, "sigmoid": torch.sigmoid,
           "gelu": F.gelu, "relu6": F.relu6, "tanh": torch.tanh}[act](z)
    _check(y, ref, tol=2e-2 if dtype == torch.bfloat16 else 6e-3)


@pytest.mark.parametrize("cfg", [
    # n, h, w, cin, cout, act, expected variant (1 streamed weights, 2 resident weights, 4 streamed on a CTA pair)
    (2, 16, 16, 64, 64, "silu", 2),
    (2, 32, 24, 48, 48, "silu", 2),
    (1, 33, 21, 32, 40, None, 2),          # ragged edges in both directions
    (2, 16, 16, 96, 96, "relu", 1),        # two channel slabs -> streamed weights
    (2, 24, 16, 192, 192, "silu", 4),      # a 192-wide filter row only double-buffers when a CTA pair splits it
    (1, 16, 16, 128, 320, None, 1),        # two column tiles
    (3, 40, 40, 8, 32, "silu", 2),         # stem-like: 8 physical input channels
])
def test_conv3x3_halo_kernel(cfg):
    from fastdeploy_b200.ops.conv_gemm import ConvGemm, pack_conv_weight
    n, h, w_, cin, cout, act, variant = cfg
    torch.manual_seed(7)
    x = (torch.randn(n, h, w_, cin, device="cuda") * 0.5).half()
    w = (torch.randn(cout, cin, 3, 3, device="cuda") * (1.0 / (cin * 9) ** 0.5)).half()
    b = torch.randn(cout, device="cuda") * 0.1
    res = (torch.randn(n, h, w_, cout, device="cuda") * 0.5).half()
    y = torch.zeros(n, h, w_, cout, device="cuda", dtype=torch.float16)
    op = ConvGemm(x, pack_conv_weight(w, torch.float16), y, in_shape=(n, h, w_, cin), out_hw=(h, w_), cout=cout,
                  kernel=(3, 3), stride=1, pad=(1, 1), bias=b, residual=res, res_mode=2, act=act, halo_mode=1)
    assert op.info()["variant"] == variant
    for _ in range(2):                      # the persistent pipeline must also be right on reuse
        op.launch()
    op.status.check()
    _check(y, _ref_conv(x, w, b, 1, 1, act, res, 2))


@pytest.mark.parametrize("y_tma_mode", [0, 1])
@pytest.mark.parametrize("cfg", [(2, 20, 20, 64, 192, 3), (1, 33, 47, 32, 40, 3), (2, 16, 16, 128, 320, 1),
                                 (2, 24, 24, 64, 68, 3), (1, 40, 40, 96, 96, 3)])
def test_conv_output_paths_agree(cfg, y_tma_mode):
    """Direct 16-byte stores and staged TMA tensor stores (ragged tiles, channel tails, concat slices)."""
    from fastdeploy_b200.ops.conv_gemm import ConvGemm, pack_conv_weight
    n, h, w_, cin, cout, k = cfg
    torch.manual_seed(8)
    x = (torch.randn(n, h, w_, cin, device="cuda") * 0.5).half()
    w = (torch.randn(cout, cin, k, k, device="cuda") * (1.0 / (cin * k * k) ** 0.5)).half()
    b = torch.randn(cout, device="cuda") * 0.1
    total = (cout + 7) // 8 * 8 + 64
    ybuf = torch.zeros(n, h, w_, total, device="cuda", dtype=torch.float16)
    res = (torch.randn(n, h, w_, cout, device="cuda") * 0.5).half()
    op = ConvGemm(x, pack_conv_weight(w, torch.float16), ybuf[..., 64:64 + cout], in_shape=(n, h, w_, cin),
                  out_hw=(h, w_), cout=cout, kernel=(k, k), stride=1, pad=(k // 2, k // 2), bias=b, residual=res,
                  res_mode=2, act="silu", y_ld=total, y_tma_mode=y_tma_mode)
    for _ in range(3):
        op.launch()
    op.status.check()
    _check(ybuf[..., 64:64 + cout], _ref_conv(x, w, b, 1, k // 2, "silu", res, 2))
    assert float(ybuf[..., :64].abs().max()) == 0.0
    if ybuf.shape[-1] > 64 + cout:
        assert float(ybuf[..., 64 + cout:].abs().max()) == 0.0


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("act", [None, "relu", "silu"])
@pytest.mark.parametrize("hw", [(64, 96), (37, 51)])
def test_stem_conv_matches_fp32_reference(dtype, act, hw):
    from fastdeploy_b200.ops.stem_conv import StemConv
    torch.manual_seed(3)
    n, (h, w) = 3, hw
    x = torch.zeros(n, h, w, 8, device="cuda", dtype=dtype)
    x[..., :3] = torch.randn(n, h, w, 3, device="cuda").to(dtype)
    x[..., 3:] = 7.0        # padding channels must not leak into the result
    wt = torch.randn(32, 3, 3, 3) * 0.2
    b = torch.randn(32)
    ho, wo = (h - 1) // 2 + 1, (w - 1) // 2 + 1
    y = torch.empty(n, ho, wo, 32, device="cuda", dtype=dtype)
    op = StemConv(x, wt.numpy(), y, n=n, h=h, w=w, bias=b.numpy(), act=act)
    op.launch()
    torch.cuda.synchronize()
    ref = torch.nn.functional.conv2d(x[..., :3].float().permute(0, 3, 1, 2), wt.cuda(), b.cuda(), stride=2, padding=1)
    if act == "relu":
        ref = torch.relu(ref)
    elif act == "silu":
        ref = torch.nn.functional.silu(ref)
    ref = ref.permute(0, 2, 3, 1)
    tol = 2e-2 if dtype == torch.bfloat16 else 4e-3
    err = (y.float() - ref).abs().max().item()
    assert err <= tol * max(1.0, ref.abs().max().item()), err


@pytest.mark.parametrize("m,k,n", [(256, 256, 128), (1000, 1280, 320), (4096, 5120, 1280)])
@pytest.mark.parametrize("act", [None, "gelu"])
def test_fp8_linear_matches_quantised_reference(m, k, n, act):
    """fp8 GEMM against an fp32 product of the same quantised operands (exact up to accumulation order), and
    against the unquantised product within e4m3's precision."""
    from fastdeploy_b200.ops.conv_gemm import linear_fp8, quantize_rows_e4m3
    torch.manual_seed(0)
    x = torch.randn(m, k, device="cuda") * 0.7
    w = torch.randn(n, k, device="cuda") * 0.05
    b = torch.randn(n, device="cuda")
    y = linear_fp8(x, w, b, act=act).float()
    xq, sa = quantize_rows_e4m3(x)
    wq, sb = quantize_rows_e4m3(w)
    ref_q = (xq.float() @ wq.float().T) * sa[:, None] * sb[None, :] + b
    ref = x @ w.T + b
    if act == "gelu":
        ref_q, ref = torch.nn.functional.gelu(ref_q), torch.nn.functional.gelu(ref)
    scale = ref.abs().max().item()
    assert (y - ref_q).abs().max().item() <= 1.5e-2 * scale        # bf16 output rounding
    assert (y - ref).abs().max().item() <= 8e-2 * scale            # e4m3 quantisation error
