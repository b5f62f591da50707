"""Device post-processing kernels against their host restatements."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_row_topk_matches_sorted_reference_with_ties():
    from fastdeploy_b200.ops.postproc import row_topk
    g = torch.Generator().manual_seed(0)
    x = torch.randn(37, 1000, generator=g)
    x[3, 10] = x[3, 700] = 9.0          # a tie: the lower index must come first
    for dt in (torch.float32, torch.float16, torch.bfloat16):
        xd = x.to(dt).cuda()
        val, idx = row_topk(xd, 5)
        ref = xd.float().cpu().numpy()
        order = np.lexsort((np.arange(1000)[None].repeat(37, 0), -ref), axis=1)[:, :5]
        assert np.array_equal(idx.cpu().numpy(), order.astype(np.int32))
        assert np.array_equal(val.cpu().numpy(), np.take_along_axis(ref, order, 1))


def test_ctc_decode_matches_host():
    from fastdeploy_b200.ops.postproc import ctc_greedy_decode_device, ctc_texts
    from fastdeploy_b200.vision.ocr import ctc_greedy_decode
    rng = np.random.default_rng(1)
    probs = rng.random((9, 70, 97)).astype(np.float32)
    # long runs of repeats and blanks
    for b in range(9):
        for t in range(70):
            k = [0, 5, 5, 7, 0, 0, 7, 9][(t // (b + 1)) % 8]
            probs[b, t, k] += 2.0
    labels = ["#"] + [chr(33 + i) for i in range(95)] + [" "]
    texts_ref, scores_ref = ctc_greedy_decode(probs, labels)
    ids, lens, sc = ctc_greedy_decode_device(torch.from_numpy(probs).cuda())
    texts, scores = ctc_texts(ids, lens, sc, labels)
    assert texts == texts_ref
    assert np.allclose(scores, scores_ref, atol=1e-5)


def test_rotate_crop_batch_matches_opencv():
    cv2 = pytest.importorskip("cv2")
    from fastdeploy_b200.ops.postproc import rotate_crop_batch
    from fastdeploy_b200.vision.ocr import get_rotate_crop_image
    yy, xx = np.mgrid[0:240, 0:320].astype(np.float32)
    img = np.stack([(np.sin(xx / 17) * 100 + 128), (np.cos(yy / 13) * 100 + 128), (xx + yy) / 560 * 255], -1)
    img = np.clip(img, 0, 255).astype(np.uint8)
    boxes = [[20, 30, 200, 40, 198, 90, 18, 80], [250, 10, 290, 12, 288, 200, 248, 198], [5, 5, 60, 5, 60, 25, 5, 25]]
    out, sizes = rotate_crop_batch(torch.from_numpy(img).cuda(), boxes)
    out = out.cpu().numpy()
    for i, box in enumerate(boxes):
        ref = get_rotate_crop_image(img, box)
        w, h = sizes[i]
        assert ref.shape[:2] == (h, w)
        diff = np.abs(out[i, :h, :w].astype(np.int32) - ref.astype(np.int32))
        # OpenCV interpolates with 5-bit fixed-point weights: allow a few grey levels
        assert diff.max() <= 6 and diff.mean() < 1.0, (i, diff.max(), diff.mean())


def test_hard_voxelize_matches_host():
    from fastdeploy_b200.ops.postproc import hard_voxelize_device
    from fastdeploy_b200.vision.perception import hard_voxelize
    rng = np.random.default_rng(2)
    pts = rng.uniform([-2, -2, -1, 0], [12, 12, 3, 1], size=(5000, 4)).astype(np.float32)
    vs, rg = [0.5, 0.5, 4.0], [0, 0, -1, 10, 10, 3]
    for max_points, max_voxels in ((8, 1000), (4, 150)):
        v_ref, c_ref, n_ref = hard_voxelize(pts, vs, rg, max_points, max_voxels)
        v, c, n = hard_voxelize_device(torch.from_numpy(pts).cuda(), vs, rg, max_points, max_voxels)
        assert np.array_equal(c.cpu().numpy(), c_ref)
        assert np.array_equal(n.cpu().numpy(), n_ref)
        assert np.array_equal(v.cpu().numpy(), v_ref)


def test_nvjpeg_decodes_into_a_device_buffer():
    import cv2
    from fastdeploy_b200.vision.common.image_decoder import ImageDecoder, ImageDecoderLib, jpeg_info, nvjpeg_available
    if not nvjpeg_available():
        pytest.skip("libnvjpeg is not installed")
    yy, xx = np.mgrid[0:120, 0:200]
    im = np.stack([(xx * 1.2) % 256, (yy * 2.0) % 256, (xx + yy) % 256], -1).astype(np.uint8)
    im = cv2.GaussianBlur(im, (0, 0), 1.5)
    ok, enc = cv2.imencode(".jpg", im, [cv2.IMWRITE_JPEG_QUALITY, 95])
    assert ok and jpeg_info(enc.tobytes()) == (120, 200, 3)
    host = ImageDecoder(ImageDecoderLib.OPENCV).decode(enc.tobytes())
    dec = ImageDecoder(ImageDecoderLib.NVJPEG)
    dev = dec.decode(enc.tobytes())
    assert dev.is_cuda and tuple(dev.shape) == (120, 200, 3)
    diff = np.abs(dev.cpu().numpy().astype(np.int32) - host.astype(np.int32))
    # IDCT and chroma up-sampling differ slightly between decoders, most at sharp colour edges
    assert diff.mean() < 1.5 and np.percentile(diff, 99) <= 8
    # into the middle of a larger staging buffer, RGB order
    buf = torch.zeros(3 * 120 * 200 * 3, dtype=torch.uint8, device="cuda")
    h, w = dec.decode_into(enc.tobytes(), buf[120 * 200 * 3:], bgr=False)
    torch.cuda.synchronize()
    got = buf[120 * 200 * 3:2 * 120 * 200 * 3].view(h, w, 3).cpu().numpy()
    assert np.abs(got[:, :, ::-1].astype(np.int32) - host.astype(np.int32)).mean() < 1.0
    assert int(buf[:120 * 200 * 3].sum()) == 0 and int(buf[2 * 120 * 200 * 3:].sum()) == 0
    with pytest.raises(ValueError):
        dec.decode(b"not a jpeg")
