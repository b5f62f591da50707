"""FDTensor and the function library against literal expectations (mirrors tests/core/test_fd_tensor.cc
and tests/function/test_*.cc of the reference)."""
import numpy as np
import pytest


def test_fd_tensor_basics():
    from fastdeploy_b200.core.fd_tensor import FDTensor
    from fastdeploy_b200.core.types import FDDataType
    t = FDTensor("x")
    t.allocate([2, 3], FDDataType.FP32)
    assert t.numel() == 6 and t.nbytes() == 24
    held = t.nbytes_allocated()
    t.resize([1, 2])                       # shrinking keeps the storage
    assert t.nbytes_allocated() == held
    t.resize([4, 4])
    assert t.nbytes_allocated() == 64
    a = np.arange(6, dtype=np.int64).reshape(2, 3)
    t.set_data([2, 3], FDDataType.INT64, a)
    assert np.array_equal(t.cpu_data(), a)
    assert t.reshape([3, -1]) and t.shape == [3, 2]
    assert not t.reshape([4, 2])
    t.expand_dim(0)
    assert t.shape == [1, 3, 2]
    t.squeeze(0)
    ext = np.ones((2, 2), np.float32)
    b = FDTensor.from_numpy(ext, copy=False)
    ext[0, 0] = 5
    assert b.cpu_data()[0, 0] == 5          # borrowed
    b.stop_sharing()
    ext[0, 0] = 7
    assert b.cpu_data()[0, 0] == 5
    c = b.clone()
    assert c.cpu_data().tolist() == b.cpu_data().tolist()
    assert "mean=" in c.print_info()


def test_elementwise_broadcast_and_reduce():
    import fastdeploy_b200.function as fn
    x = np.array([[1., 2., 3.], [4., 5., 6.]], np.float32)
    y = np.array([10., 20., 30.], np.float32)
    assert fn.add(x, y).cpu_data().tolist() == [[11, 22, 33], [14, 25, 36]]
    assert fn.divide(np.array([7, -7]), np.array([2, 2])).cpu_data().tolist() == [3, -3]
    assert fn.sum(x, [1]).cpu_data().tolist() == [6, 15]
    assert fn.mean(x, [0], keep_dim=True).cpu_data().tolist() == [[2.5, 3.5, 4.5]]
    assert fn.max(x, reduce_all=True).cpu_data().item() == 6
    assert fn.prod(x, [1]).cpu_data().tolist() == [6, 120]
    assert fn.all(np.array([[1, 0], [1, 1]]), [1]).cpu_data().tolist() == [False, True]
    assert fn.any(np.array([[0, 0], [0, 1]]), [1]).cpu_data().tolist() == [False, True]
    assert fn.argmax(x, 1).cpu_data().tolist() == [2, 2]
    assert fn.argmin(x, 0, keep_dim=True).cpu_data().tolist() == [[0, 0, 0]]


def test_shape_functions():
    import fastdeploy_b200.function as fn
    x = np.arange(24, dtype=np.float32).reshape(2, 3, 4)
    assert fn.transpose(x, [2, 0, 1]).shape == [4, 2, 3]
    assert fn.concat([x, x], 1).shape == [2, 6, 4]
    parts = fn.split(x, [1, -1], axis=2)
    assert [p.shape for p in parts] == [[2, 3, 1], [2, 3, 3]]
    assert fn.slice(x, [0, 2], [1, 1], [2, 3]).cpu_data().tolist() == x[1:2, :, 1:3].tolist()
    assert fn.slice(x, [1], [2]).shape == [2, 4]
    assert fn.tile(np.array([[1, 2]]), [2, 2]).cpu_data().tolist() == [[1, 2, 1, 2], [1, 2, 1, 2]]
    assert fn.pad(np.ones((1, 2), np.float32), [1, 0, 0, 2], 9).cpu_data().tolist() == [[9, 9, 9, 9], [1, 1, 9, 9]]
    assert fn.cumprod(np.array([1., 2., 3.]), 0).cpu_data().tolist() == [1, 2, 6]
    assert fn.clip(np.array([-1., 0.5, 2.]), 0, 1).cpu_data().tolist() == [0, 0.5, 1]
    assert fn.linspace(0, 1, 5).cpu_data().tolist() == [0, 0.25, 0.5, 0.75, 1.0]
    assert fn.full(3, [2]).cpu_data().tolist() == [3, 3]


def test_math_sort_softmax_quantile_gather():
    import fastdeploy_b200.function as fn
    from fastdeploy_b200.core.types import FDDataType
    x = np.array([[3., 1., 2.], [0., 5., 4.]], np.float32)
    v, i = fn.sort(x, 1, descending=True)
    assert v.cpu_data().tolist() == [[3, 2, 1], [5, 4, 0]] and i.cpu_data().tolist() == [[0, 2, 1], [1, 2, 0]]
    assert fn.argsort(x, 1).cpu_data().tolist() == [[1, 2, 0], [0, 2, 1]]
    s = fn.softmax(x, 1).cpu_data()
    assert np.allclose(s.sum(1), 1) and np.allclose(s[0], np.exp(x[0]) / np.exp(x[0]).sum(), atol=1e-6)
    q = fn.quantile(np.array([1., 2., 3., 4.]), [0.5, 1.0], [0]).cpu_data()
    assert np.allclose(q, [2.5, 4.0])
    g = fn.gather_along_axis(x, np.array([[0], [2]]), 1).cpu_data()
    assert g.tolist() == [[3.], [4.]]
    sc = fn.scatter_along_axis(np.zeros((2, 3), np.float32), np.array([[1], [0]]), np.array([[7.], [8.]], np.float32), 1)
    assert sc.cpu_data().tolist() == [[0, 7, 0], [8, 0, 0]]
    assert fn.cast(x, FDDataType.INT32).cpu_data().dtype == np.int32
    assert fn.isnan(np.array([1., np.nan])).cpu_data().tolist() == [False, True]
    assert fn.isinf(np.array([1., np.inf])).cpu_data().tolist() == [False, True]
    assert fn.isfinite(np.array([1., np.inf, np.nan])).cpu_data().tolist() == [True, False, False]
    assert np.allclose(fn.sqrt(np.array([4.])).cpu_data(), 2) and np.allclose(fn.exp(np.array([0.])).cpu_data(), 1)
    assert fn.round(np.array([1.4, 2.6])).cpu_data().tolist() == [1, 3]
    assert fn.floor(np.array([1.5])).cpu_data().tolist() == [1] and fn.ceil(np.array([1.5])).cpu_data().tolist() == [2]
    a = fn.gaussian_random([1000], 1.0, 2.0, seed=3).cpu_data()
    assert abs(a.mean() - 1.0) < 0.3 and abs(a.std() - 2.0) < 0.3
    assert np.array_equal(a, fn.gaussian_random([1000], 1.0, 2.0, seed=3).cpu_data())


def test_scalar_ue8m0_timecounter_and_backend_tables():
    import math
    import time
    import fastdeploy_b200 as fd
    from fastdeploy_b200.core.scalar import Scalar, ue8m0_from_float, ue8m0_to_float
    from fastdeploy_b200.core.types import supported
    from fastdeploy_b200.utils.perf import TimeCounter
    assert Scalar(3).dtype == fd.FDDataType.INT64 and Scalar(3).to(int) == 3 and Scalar(2.5).to(float) == 2.5
    assert Scalar(True).dtype == fd.FDDataType.BOOL and Scalar(7.9, fd.FDDataType.INT32).to(int) == 7
    assert Scalar("-inf").to(float) == -math.inf and math.isnan(Scalar("nan").to(float))
    assert Scalar(2 ** 40 + 1).to(int) == 2 ** 40 + 1
    with pytest.raises(ValueError):
        Scalar("twelve")
    # ue8m0: powers of two are exact, everything else rounds up so a scaled block cannot overflow
    assert ue8m0_to_float(ue8m0_from_float(1.0)) == 1.0 and ue8m0_to_float(ue8m0_from_float(0.25)) == 0.25
    assert ue8m0_to_float(ue8m0_from_float(3.0)) == 4.0 and ue8m0_to_float(ue8m0_from_float(0.3)) == 0.5
    assert ue8m0_from_float(float("nan")) == 255 and math.isnan(ue8m0_to_float(255))
    t = TimeCounter()
    t.start()
    time.sleep(0.02)
    t.end()
    assert 0.015 < t.duration() < 0.5
    assert fd.Backend.NATIVE in fd.get_available_backends() and fd.is_backend_available(fd.Backend.TRT)
    assert supported(fd.ModelFormat.ONNX, fd.Backend.ORT) and not supported(fd.ModelFormat.ONNX, fd.Backend.PDINFER)
    assert supported(fd.Device.GPU, fd.Backend.TRT)
