"""Allocation-free global average pooling, called through its exported C symbol.

Some users of the C ABI cannot allocate device memory when they call in - plugin code inside
a host application whose memory budget is fixed at start-up, latency-critical loops where
cudaMalloc's device-wide synchronisation is unacceptable, C programs without a caching
allocator. For them ``fdb_global_avgpool_noalloc`` keeps its scratch in a fixed array inside
the library. The test checks it against the regular entry point (caller-allocated scratch) on
two calls in a row, the second one smaller, so stale scratch contents would show up.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

MAX_SCRATCH_FLOATS = 1 << 20


def _lib():
    from fastdeploy_b200 import _native
    lib = _native.kernels()
    fn = lib.fdb_global_avgpool_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                   ctypes.c_longlong, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    lib.fdb_global_avgpool_noalloc_strerror.restype = ctypes.c_char_p
    lib.fdb_global_avgpool_noalloc_strerror.argtypes = [ctypes.c_int]
    return lib


def _regular(x, n, hw, c, ld, splits, out_dtype):
    from fastdeploy_b200.ops import nhwc
    scratch = torch.empty(n * splits * c, device="cuda")
    out = torch.zeros(n, c, device="cuda", dtype=out_dtype)
    for op in nhwc.global_avgpool(x, out, scratch, n=n, hw=hw, c=c, x_ld=ld, splits=splits):
        op.launch()
    return out


def test_noalloc_matches_regular_entry_point_twice():
    lib = _lib()
    torch.manual_seed(0)
    stream = torch.cuda.current_stream().cuda_stream
    cases = [(4, 24 * 20, 96, 128, 5, torch.float16, torch.float32),
             (2, 7 * 9, 64, 64, 2, torch.bfloat16, torch.bfloat16)]
    for n, hw, c, ld, splits, dt, odt in cases:
        buf = torch.randn(n, hw, ld, device="cuda").to(dt)
        x = buf[..., ld - c:]
        want = _regular(x, n, hw, c, ld, splits, odt)
        got = torch.zeros(n, c, device="cuda", dtype=odt)
        code = {torch.float16: 0, torch.bfloat16: 1, torch.float32: 2}[odt]
        rc = lib.fdb_global_avgpool_noalloc(x.data_ptr(), got.data_ptr(), n, hw, c, ld, 0, splits,
                                            int(dt == torch.bfloat16), code, c, ctypes.c_void_p(stream))
        assert rc == 0, lib.fdb_global_avgpool_noalloc_strerror(rc)
        torch.cuda.synchronize()
        err = (got.float() - want.float()).abs().max().item()
        assert err <= 2e-3, err
        ref = x.float().mean(1)
        assert (got.float() - ref).abs().max().item() <= (2e-3 if odt == torch.float32 else 2e-2)


def test_noalloc_rejects_oversize_and_bad_arguments():
    lib = _lib()
    x = torch.zeros(8, device="cuda", dtype=torch.float16)
    out = torch.zeros(8, device="cuda")
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    n, splits, c = 64, 64, 512                       # 2 Mi floats of scratch would be needed
    assert n * splits * c > MAX_SCRATCH_FLOATS
    rc = lib.fdb_global_avgpool_noalloc(x.data_ptr(), out.data_ptr(), n, 4096, c, c, 0, splits, 0, 2, c, stream)
    assert rc == 2 and b"exceeds" in lib.fdb_global_avgpool_noalloc_strerror(rc)
    rc = lib.fdb_global_avgpool_noalloc(x.data_ptr(), out.data_ptr(), 1, 16, 12, 16, 0, 1, 0, 2, 12, stream)
    assert rc == 1                                   # channels not a multiple of 8
    rc = lib.fdb_global_avgpool_noalloc(None, out.data_ptr(), 1, 16, 8, 8, 0, 1, 0, 2, 8, stream)
    assert rc == 1
    # host-side rejections, nothing is launched: an image stride that would misalign every image after the
    # first, one shorter than an image, a row pitch below the channel count, an output type that does not exist
    big = torch.zeros(4 * 16 * 16 + 64, device="cuda", dtype=torch.float16)
    for args in ((2, 16, 8, 16, 16 * 16 + 4, 1, 0, 2, 8), (2, 16, 8, 16, 16 * 8, 1, 0, 2, 8),
                 (2, 16, 8, 16, -256, 1, 0, 2, 8), (1, 16, 16, 8, 0, 1, 0, 2, 16), (1, 16, 8, 8, 0, 1, 0, 3, 8),
                 (1, 16, 8, 8, 0, 1, 0, 2, 4)):
        rc = lib.fdb_global_avgpool_noalloc(big.data_ptr(), out.data_ptr(), *args, stream)
        assert rc == 1, args
    assert b"x_n_stride" in lib.fdb_global_avgpool_noalloc_strerror(1)
    rc = lib.fdb_global_avgpool_noalloc(big.data_ptr() + 2, out.data_ptr(), 1, 16, 8, 8, 0, 1, 0, 2, 8, stream)
    assert rc == 1                                   # x not 16-byte aligned
    torch.cuda.synchronize()


def test_noalloc_with_padded_image_stride():
    """Images that sit further apart than hw * x_ld (a batch carved out of a larger buffer)."""
    lib = _lib()
    torch.manual_seed(1)
    n, hw, c, ld, splits = 3, 5 * 7, 32, 40, 3
    stride = hw * ld + 64
    buf = torch.randn(n * stride, device="cuda").to(torch.float16)
    x = torch.as_strided(buf, (n, hw, c), (stride, ld, 1))
    got = torch.zeros(n, c, device="cuda")
    rc = lib.fdb_global_avgpool_noalloc(x.data_ptr(), got.data_ptr(), n, hw, c, ld, stride, splits, 0, 2, c,
                                        ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0, lib.fdb_global_avgpool_noalloc_strerror(rc)
    torch.cuda.synchronize()
    assert (got - x.float().mean(1)).abs().max().item() <= 2e-3
