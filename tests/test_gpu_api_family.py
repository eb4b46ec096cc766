"""The callers next to sort/argsort in the reference's API module: sort_complex, partition,
argpartition (full sorts there too) and lexsort, each against NumPy."""
import numpy as np
import pytest

import cupynumeric_b200 as num

pytestmark = pytest.mark.gpu


def test_sort_complex(cuda_device):
    rng = np.random.default_rng(1)
    for a in (rng.integers(-50, 50, 300).astype(np.int16), rng.integers(-50, 50, 300).astype(np.int64),
              rng.standard_normal(300).astype(np.float32),
              (rng.integers(-5, 5, 300) + 1j * rng.integers(-5, 5, 300)).astype(np.complex64)):
        got = num.sort_complex(a).to_numpy()
        want = np.sort_complex(a)
        assert got.dtype == want.dtype and np.array_equal(got, want), a.dtype


def test_partition_and_argpartition(cuda_device):
    rng = np.random.default_rng(2)
    a = rng.integers(-100, 100, (6, 50)).astype(np.int32)
    for axis in (0, 1, -1):
        for kth in (0, 3, -1, [1, 4]):
            p = num.partition(a, kth, axis=axis).to_numpy()
            ip = num.argpartition(a, kth, axis=axis).to_numpy()
            srt = np.sort(a, axis=axis)
            for k in np.atleast_1d(kth):
                assert np.array_equal(np.take(p, k, axis=axis), np.take(srt, k, axis=axis))
            assert np.array_equal(np.take_along_axis(a, ip, axis=axis), p)
    with pytest.raises(ValueError):
        num.partition(a, 50, axis=1)
    with pytest.raises(ValueError):
        num.argpartition(a, 0, axis=2)


def test_lexsort(cuda_device):
    rng = np.random.default_rng(3)
    k1 = rng.integers(0, 4, 2000).astype(np.int32)
    k2 = rng.integers(0, 3, 2000).astype(np.float64)
    k2[::97] = np.nan
    k2[5::101] = np.inf
    k3 = rng.integers(0, 2, 2000).astype(np.int8)
    assert np.array_equal(num.lexsort((k1, k2, k3)).to_numpy(), np.lexsort((k1, k2, k3)))
    m1, m2 = rng.integers(0, 3, (7, 40)), rng.integers(0, 3, (7, 40))
    for axis in (0, 1):
        assert np.array_equal(num.lexsort((m1, m2), axis=axis).to_numpy(), np.lexsort((m1, m2), axis=axis))
    with pytest.raises(TypeError):
        num.lexsort((k1, k2), axis=None)
    with pytest.raises(ValueError):
        num.lexsort((k1, k2[:10]))


def test_unique(cuda_device):
    rng = np.random.default_rng(4)
    dtypes = [np.bool_, np.int8, np.int16, np.int32, np.int64, np.uint8, np.uint16, np.uint32, np.uint64,
              np.float16, np.float32, np.float64]
    for dtype in dtypes:
        for n in (0, 1, 5, 4096, 4097, 300_000):
            raw = rng.integers(-40, 40, n)
            a = (np.abs(raw) if np.dtype(dtype).kind in "ub" else raw).astype(dtype)
            if np.dtype(dtype).kind == "f" and n > 4:
                a[::5] = np.nan
                a[1::7] = -0.0
                a[2::7] = 0.0
            got = num.unique(a).to_numpy()
            want = np.unique(a)
            assert got.shape == want.shape and np.array_equal(got, want, equal_nan=np.dtype(dtype).kind == "f"), (dtype, n)
    c = (rng.integers(-6, 6, 50_000) + 1j * rng.integers(-6, 6, 50_000)).astype(np.complex64)
    assert np.array_equal(num.unique(c).to_numpy(), np.unique(c))        # complex64: one 8-byte key
    m = rng.integers(0, 10, (30, 40)).astype(np.int32)
    assert np.array_equal(num.unique(m).to_numpy(), np.unique(m))
    with pytest.raises(NotImplementedError):
        num.unique(m, return_counts=True)
    with pytest.raises(NotImplementedError):
        num.unique(m, axis=0)
