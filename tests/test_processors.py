"""Processor semantics and fused-vs-unfused equivalence (mirrors tests/vision_preprocess/* of the reference)."""
import numpy as np
import pytest

from fastdeploy_b200.vision.common import (BGR2RGB, Cast, CenterCrop, FDMat, HWC2CHW, LimitByStride, Normalize,
                                           NormalizeAndPermute, Pad, PadToSize, ProcessorManager, Resize,
                                           ResizeByShort, StridePad, chain_geometry, fuse_transforms)


def _img(h=64, w=64, seed=0):
    return np.random.RandomState(seed).randint(0, 256, (h, w, 3), dtype=np.uint8)


def test_normalize_and_permute_equals_normalize_plus_hwc2chw():
    mean, std = [0.5, 0.4, 0.3], [0.2, 0.3, 0.4]
    a = FDMat(_img())
    Normalize(mean, std)(a)
    HWC2CHW()(a)
    b = FDMat(_img())
    NormalizeAndPermute(mean, std)(b)
    assert a.layout == b.layout == "CHW" and np.array_equal(a.mat, b.mat)
    ref = (_img().astype(np.float32) / 255.0 - np.float32(mean)) / np.float32(std)
    assert np.allclose(a.mat.transpose(1, 2, 0), ref, atol=1e-5)


def test_fuse_transforms():
    chain = [BGR2RGB(), Resize(32, 32), Normalize([0.5] * 3, [0.5] * 3), Cast("float"), HWC2CHW()]
    fused = fuse_transforms(chain)
    assert [type(p).__name__ for p in fused] == ["Resize", "Normalize", "HWC2CHW"] or \
        [type(p).__name__ for p in fused] == ["Resize", "NormalizeAndPermute"]
    assert fused[1].swap_rb is True
    a, b = FDMat(_img()), FDMat(_img())
    for p in chain:
        p(a)
    for p in fused:
        p(b)
    assert np.allclose(a.mat, b.mat, atol=1e-6)


def test_geometric_processors():
    m = FDMat(_img(50, 70))
    ResizeByShort(100, 1, True, [120, 120])(m)
    assert (m.height(), m.width()) == (86, 120)          # limited by max_hw on the long side
    CenterCrop(64, 64)(m)
    assert m.mat.shape == (64, 64, 3)
    StridePad(48, [1, 2, 3])(m)
    assert m.mat.shape == (96, 96, 3) and m.mat[95, 95].tolist() == [1, 2, 3]
    PadToSize(100, 128, [0, 0, 0])(m)
    assert m.mat.shape == (128, 100, 3)
    LimitByStride(32)(m)
    assert m.mat.shape == (128, 96, 3)
    Pad(1, 2, 3, 4, [9, 9, 9])(m)
    assert m.mat.shape == (131, 103, 3) and m.mat[0, 0].tolist() == [9, 9, 9]
    with pytest.raises(ValueError):
        CenterCrop(500, 500)(FDMat(_img()))


def test_manager_batches_and_pads():
    mgr = ProcessorManager()
    mgr.processors = [ResizeByShort(32), NormalizeAndPermute([0.5] * 3, [0.5] * 3)]
    out = mgr.run([_img(40, 80), _img(64, 64, 1)])[0]
    assert out.shape == (2, 3, 32, 64) and out.dtype == np.float32
    assert np.all(out[1, :, :, 32:] == 0)


def test_chain_geometry_folding():
    g = chain_geometry([BGR2RGB(), Resize(640, 640, interp=2), NormalizeAndPermute([0] * 3, [1] * 3)], 1080, 1920)
    assert g["rh"] == g["rw"] == 640 and g["interp"] == 2 and g["swap_rb"] and g["chw"]
    assert np.allclose(g["alpha"], [1 / 255] * 3)
    assert chain_geometry([CenterCrop(10, 10)], 20, 20) is None
