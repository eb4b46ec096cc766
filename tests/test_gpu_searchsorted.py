"""SEARCHSORTED against numpy.searchsorted (the reference's own test oracle,
tests/integration/test_searchsorted.py): all radix dtypes, both sides, duplicates, values outside
the range, empty inputs, scalars, N-D value arrays, type promotion and ``sorter``."""
import numpy as np
import pytest

import cupynumeric_b200 as num

pytestmark = pytest.mark.gpu

DTYPES = [np.bool_, np.int8, np.int16, np.int32, np.int64, np.uint8, np.uint16, np.uint32, np.uint64,
          np.float16, np.float32, np.float64]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("side", ["left", "right"])
def test_searchsorted_matches_numpy(cuda_device, dtype, side):
    rng = np.random.default_rng(3)
    for n, m in ((0, 5), (1, 7), (1000, 333), (100_000, 20_000)):
        raw = rng.integers(-60, 60, n)
        a = np.sort((np.abs(raw) if np.dtype(dtype).kind in "ub" else raw).astype(dtype))
        vraw = rng.integers(-80, 80, m)
        v = (np.abs(vraw) if np.dtype(dtype).kind in "ub" else vraw).astype(dtype)
        got = num.searchsorted(a, v, side=side).to_numpy()
        assert got.dtype == np.int64
        assert np.array_equal(got, np.searchsorted(a, v, side=side)), (np.dtype(dtype), side, n)


def test_searchsorted_complex64(cuda_device):
    rng = np.random.default_rng(5)
    a = np.sort((rng.integers(-9, 9, 20_000) + 1j * rng.integers(-9, 9, 20_000)).astype(np.complex64))
    v = (rng.integers(-11, 11, 3000) + 1j * rng.integers(-11, 11, 3000)).astype(np.complex64)
    for side in ("left", "right"):
        assert np.array_equal(num.searchsorted(a, v, side=side).to_numpy(), np.searchsorted(a, v, side=side))


def test_searchsorted_shapes_promotion_sorter_and_errors(cuda_device):
    rng = np.random.default_rng(4)
    a = np.sort(rng.standard_normal(5000).astype(np.float32))
    a[-3:] = np.nan                                   # NaN sorts last and is found there
    v = np.array([[-10.0, 0.0, 0.5], [np.nan, 10.0, a[17]]], dtype=np.float32)
    for side in ("left", "right"):
        assert np.array_equal(num.searchsorted(a, v, side=side).to_numpy(), np.searchsorted(a, v, side=side))
    assert num.searchsorted(a, 0.25).to_numpy() == np.searchsorted(a, 0.25)
    ai = np.arange(0, 100, 2, dtype=np.int32)
    vf = np.array([2.5, 3.0, -1.0, 99.5])
    assert np.array_equal(num.searchsorted(ai, vf).to_numpy(), np.searchsorted(ai, vf))   # int32 with float64
    unsorted = rng.integers(0, 1000, 777).astype(np.int64)
    order = np.argsort(unsorted, kind="stable")
    vv = rng.integers(-5, 1005, 100).astype(np.int64)
    assert np.array_equal(num.searchsorted(unsorted, vv, side="right", sorter=order).to_numpy(),
                          np.searchsorted(unsorted, vv, side="right", sorter=order))
    with pytest.raises(ValueError):
        num.searchsorted(np.zeros((2, 2)), 1.0)
    with pytest.raises(ValueError):
        num.searchsorted(ai, vf, sorter=np.zeros((2, 2), dtype=np.int64))
