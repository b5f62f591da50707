"""The native host function library against numpy on random strided operands, plus the reference's edge semantics."""
import numpy as np
import pytest
import torch

import fastdeploy_b200.function as fn
from fastdeploy_b200.function import native as N

DTYPES = [np.float32, np.float64, np.int32, np.int64, np.uint8]


def _arr(rng, shape, dt):
    if np.dtype(dt).kind == "f":
        return rng.standard_normal(shape).astype(dt)
    return rng.integers(0 if np.dtype(dt).kind == "u" else -20, 20, shape).astype(dt)


def _np(t):
    return t.tensor().numpy()


def test_native_library_is_the_path_taken_for_host_tensors():
    x = np.ones((2, 3), np.float32)
    assert N.usable(x) and fn._np(x) is not None and fn._np(torch.ones(2, dtype=torch.float16)) is None


@pytest.mark.parametrize("dt", DTYPES)
def test_elementwise_and_layout_functions_match_numpy(dt):
    rng = np.random.default_rng(1)
    a = _arr(rng, (3, 4, 5), dt)
    b = _arr(rng, (4, 1), dt)
    b[b == 0] = 3
    view = a.transpose(2, 0, 1)[::2]                      # a strided operand
    assert np.array_equal(_np(fn.add(view, 1 * view)), view + view)
    assert np.array_equal(_np(fn.subtract(a, b)), a - b) and np.array_equal(_np(fn.multiply(a, b)), a * b)
    assert np.array_equal(_np(fn.maximum(a, b)), np.maximum(a, b))
    if np.dtype(dt).kind == "f":
        assert np.allclose(_np(fn.divide(a, b)), a / b)
    else:
        want = np.trunc(a.astype(np.float64) / b.astype(np.float64)).astype(dt)      # toward zero, not floor
        assert np.array_equal(_np(fn.divide(a, b)), want)
    assert np.array_equal(_np(fn.transpose(a, [2, 0, 1])), a.transpose(2, 0, 1))
    assert np.array_equal(_np(fn.concat([a, a[:, :2]], 1)), np.concatenate([a, a[:, :2]], 1))
    assert np.array_equal(_np(fn.tile(a[0], [2, 1, 3])), np.tile(a[0], [2, 1, 3]))
    assert np.array_equal(_np(fn.pad(a, [1, 0, 0, 2, 3, 3], 7)), np.pad(a, [(1, 0), (0, 2), (3, 3)], constant_values=7))
    assert np.array_equal(_np(fn.clip(a, -1, 2)), np.clip(a, -1, 2))
    assert np.array_equal(_np(fn.abs(a)), np.abs(a))
    assert np.array_equal(_np(fn.slice(a, [0, 2], [1, 1], [3, 4])), a[1:3, :, 1:4])


@pytest.mark.parametrize("dt", DTYPES)
def test_reductions_sort_and_selection_match_numpy(dt):
    rng = np.random.default_rng(2)
    a = _arr(rng, (3, 4, 5), dt)
    assert np.allclose(_np(fn.sum(a, [1])), a.sum(1)) and np.allclose(_np(fn.sum(a, [0, 2], keep_dim=True)), a.sum((0, 2), keepdims=True))
    assert np.allclose(_np(fn.mean(a, [2])), a.mean(2)) and np.array_equal(_np(fn.max(a, [1])), a.max(1))
    assert np.array_equal(_np(fn.min(a, reduce_all=True)), a.min()) and np.array_equal(_np(fn.any(a, [0])), a.any(0))
    assert np.array_equal(_np(fn.all(a, [1, 2])), a.all((1, 2)))
    small = (a[:, :2, :3] % 3 + 1).astype(dt)
    assert np.allclose(_np(fn.prod(small, [1, 2])), small.prod((1, 2)))
    assert np.array_equal(_np(fn.argmax(a, 1)), a.argmax(1)) and np.array_equal(_np(fn.argmin(a, -1, keep_dim=True)), a.argmin(-1, keepdims=True))
    assert _np(fn.argmax(a, 0, flatten=True)) == a.reshape(-1).argmax()
    v, i = fn.sort(a, 1)
    assert np.array_equal(_np(v), np.sort(a, 1, kind="stable")) and np.array_equal(_np(i), np.argsort(a, 1, kind="stable"))
    vd, idd = fn.sort(a, 2, descending=True)
    assert np.array_equal(_np(vd), np.take_along_axis(a, _np(idd), 2)) and (np.diff(_np(vd).astype(np.float64), axis=2) <= 0).all()
    idx = rng.integers(0, 4, (3, 2, 5))
    assert np.array_equal(_np(fn.gather_along_axis(a, idx, 1)), np.take_along_axis(a, idx, 1))
    vals = _arr(rng, (3, 2, 5), dt)
    idx2 = np.stack([rng.permutation(4)[:2] for _ in range(15)]).reshape(3, 5, 2).transpose(0, 2, 1)    # no duplicates
    want = a.copy()
    np.put_along_axis(want, idx2, vals, 1)
    assert np.array_equal(_np(fn.scatter_along_axis(a, idx2, vals, 1)), want)


def test_reference_edge_semantics():
    # sort is stable and descending keeps the earlier of equal keys first
    keys = np.array([2, 1, 2, 1, 2], np.int32)
    assert _np(fn.argsort(keys, 0)).tolist() == [1, 3, 0, 2, 4] and _np(fn.argsort(keys, 0, descending=True)).tolist() == [0, 2, 4, 1, 3]
    # arg-max / arg-min return the first extreme
    assert int(_np(fn.argmax(np.array([1, 5, 5, 2], np.float32), 0))) == 1 and int(_np(fn.argmin(np.array([3, 0, 0], np.int64), 0))) == 1
    # quantile interpolates linearly between order statistics, one row per q
    x = np.array([[4.0, 1.0, 3.0, 2.0], [10.0, 20.0, 30.0, 40.0]], np.float32)
    q = _np(fn.quantile(x, [0.0, 0.5, 0.9, 1.0], [1]))
    assert q.shape == (4, 2) and np.allclose(q, np.quantile(x, [0.0, 0.5, 0.9, 1.0], axis=1))
    assert _np(fn.quantile(np.array([1, 2, 3, 4], np.int32), [0.5], [0])).dtype == np.float64
    # integer division truncates toward zero; a zero divisor is refused
    assert _np(fn.divide(np.array([-7, 7, -1], np.int64), np.array([2, -2, 3], np.int64))).tolist() == [-3, -3, 0]
    with pytest.raises(ValueError):
        fn.divide(np.array([1], np.int32), np.array([0], np.int32))
    # pad order is [before_0, after_0, before_1, after_1]
    assert _np(fn.pad(np.ones((1, 2), np.float32), [0, 1, 2, 0], 5.0)).tolist() == [[5, 5, 1, 1], [5, 5, 5, 5]]
    # integer sums widen, the mean of integers is floating, round goes to even, NaN propagates through max
    assert _np(fn.sum(np.full((3,), 2 ** 30, np.int32), [0])).dtype == np.int64 and int(_np(fn.sum(np.full((3,), 2 ** 30, np.int32), [0]))) == 3 * 2 ** 30
    assert _np(fn.mean(np.array([1, 2], np.int32), [0])).dtype == np.float64
    assert _np(fn.round(np.array([0.5, 1.5, 2.5, -0.5], np.float32))).tolist() == [0.0, 2.0, 2.0, -0.0]
    assert np.isnan(_np(fn.max(np.array([1.0, np.nan, 3.0], np.float32), [0])))
    assert _np(fn.isnan(np.array([1.0, np.nan], np.float64))).tolist() == [False, True]
    assert _np(fn.isinf(np.array([np.inf, 1.0], np.float32))).dtype == np.bool_
    # soft-max and cumprod along an inner axis of a strided operand
    y = np.random.default_rng(3).standard_normal((4, 6, 3)).astype(np.float32).transpose(1, 0, 2)
    e = np.exp(y - y.max(1, keepdims=True))
    assert np.allclose(_np(fn.softmax(y, 1)), e / e.sum(1, keepdims=True), atol=1e-6)
    assert np.allclose(_np(fn.cumprod(y, 2)), np.cumprod(y, 2), rtol=1e-5)
    # casts: float -> integer truncates, anything -> bool is != 0
    assert _np(fn.cast(np.array([-1.7, 2.9], np.float32), fd_int32())).tolist() == [-1, 2]
    assert _np(fn.cast(np.array([0.0, 0.2], np.float64), fd_bool())).tolist() == [False, True]


def fd_int32():
    import fastdeploy_b200 as fd
    return fd.FDDataType.INT32


def fd_bool():
    import fastdeploy_b200 as fd
    return fd.FDDataType.BOOL


def test_float_to_integer_conversions_are_defined_for_every_input():
    """NaN, infinities and values outside the target type do not depend on the compiler's mood: NaN -> 0, the value is
    clamped to int64 and then wraps into the narrower type."""
    import fastdeploy_b200 as fd
    x = np.array([np.nan, np.inf, -np.inf, 300.7, -1.7, 1e30], np.float64)
    assert _np(fn.cast(x, fd.FDDataType.INT64)).tolist() == [0, 2 ** 63 - 1, -2 ** 63, 300, -1, 2 ** 63 - 1]
    assert _np(fn.cast(x, fd.FDDataType.UINT8)).tolist() == [0, 255, 0, 44, 255, 255]
    assert _np(fn.cast(x, fd.FDDataType.INT32)).tolist()[3:5] == [300, -1]


def test_slice_split_and_full_run_natively_and_match_torch():
    import torch
    import fastdeploy_b200 as fd
    x = np.arange(2 * 7 * 5, dtype=np.float32).reshape(2, 7, 5)
    t = torch.from_numpy(x)
    assert np.array_equal(_np(fn.slice(x, [1, 2], [1, -4], [6, 100])), x[:, 1:6, 1:5])
    assert np.array_equal(_np(fn.slice(x, [0, 2], [1, 3])), x[1, :, 3])
    assert _np(fn.slice(x, [1], [5], [2])).shape == (2, 0, 5)
    for n in (1, 2, 3, 7, 9):
        got = fn.split(x, n, axis=1)
        want = torch.chunk(t, n, dim=1)
        assert len(got) == len(want) and all(np.array_equal(_np(g), w.numpy()) for g, w in zip(got, want)), n
    got = fn.split(x, [2, -1, 1], axis=1)
    assert [g.shape[1] for g in got] == [2, 4, 1] and np.array_equal(_np(got[1]), x[:, 2:6])
    with pytest.raises(ValueError, match="add up"):
        fn.split(x, [2, 2], axis=1)
    f = fn.full(3, [2, 3], fd.FDDataType.INT32)
    assert _np(f).dtype == np.int32 and _np(f).tolist() == [[3, 3, 3], [3, 3, 3]]
    assert _np(fn.full(0.25, [], fd.FDDataType.FP64)).shape == () and float(_np(fn.full(0.25, [], fd.FDDataType.FP64))) == 0.25
    fl = fn.full_like(x, 7)
    assert _np(fl).dtype == np.float32 and _np(fl).shape == x.shape and (_np(fl) == 7).all()
    assert _np(fn.full_like(x, 1, fd.FDDataType.UINT8)).dtype == np.uint8
