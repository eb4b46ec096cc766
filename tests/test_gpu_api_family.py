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


def _assert_partitioned(p, a, k):
    """The partition property of numpy.partition for one kth, plus: p is a rearrangement of a."""
    srt = np.sort(a, kind="stable")
    k %= a.size
    bits = lambda x: x.view({1: np.uint8, 2: np.uint16, 4: np.uint32, 8: np.uint64}[x.dtype.itemsize])
    assert np.array_equal(np.sort(bits(p)), np.sort(bits(a))), "not a rearrangement of the input"
    pivot = srt[k]
    same = lambda x, y: (x == y) | (np.isnan(x) & np.isnan(y)) if a.dtype.kind == "f" else x == y
    assert same(p[k], pivot)
    if a.dtype.kind == "f":
        key = lambda x: np.where(np.isnan(x), np.inf, x)       # NaN sorts last
        nan_ok = np.isnan(pivot) or not np.isnan(p[:k]).any()
        assert nan_ok and (key(p[:k]) <= key(pivot)).all() and (key(p[k:]) >= key(pivot)).all()
    else:
        assert (p[:k] <= pivot).all() and (p[k:] >= pivot).all()


@pytest.mark.parametrize("dtype", [np.int8, np.uint16, np.float16, np.int32, np.float32, np.uint32, np.int64, np.float64, np.uint64])
def test_partition_by_selection_on_long_1d_arrays(cuda_device, dtype):
    """Arrays longer than the selection threshold never get sorted: the result has the partition
    property (and only that)."""
    rng = np.random.default_rng(np.dtype(dtype).itemsize + 40)
    n = 300_000
    if np.dtype(dtype).kind == "f":
        a = rng.standard_normal(n).astype(dtype)
        a[::1000] = np.nan
        a[1::777] = -0.0
        a[2::777] = 0.0
        a[3::500] = a[3]                       # a run of duplicates
    else:
        info = np.iinfo(dtype)
        a = rng.integers(max(info.min, -5000), min(info.max, 5000), n).astype(dtype)
    for kth in (0, 1, n // 3, n // 2, n - 2, n - 1, -5):
        p = num.partition(a, kth).to_numpy()
        _assert_partitioned(p, a, kth)
        ip = num.argpartition(a, kth).to_numpy()
        assert np.array_equal(np.sort(ip), np.arange(n)), "not a permutation"
        _assert_partitioned(a[ip], a, kth)
    # axis=None on a 2-D array flattens first
    m = a[: 200 * 500].reshape(200, 500)
    _assert_partitioned(num.partition(m, 777, axis=None).to_numpy(), m.reshape(-1), 777)
    # all keys equal; and kth inside a long run of one value
    c = np.full(50_000, 7, dtype=dtype)
    _assert_partitioned(num.partition(c, 12_345).to_numpy(), c, 12_345)


def test_selection_really_skips_the_sort(cuda_device):
    """No radix pass runs for a long 1-D partition."""
    from cupynumeric_b200 import _lib

    lib = _lib.lib()
    a = np.random.default_rng(0).integers(0, 1 << 30, 1 << 20).astype(np.int32)
    d = num.array(a)
    before = lib.b2s_launch_count(_lib.K_SWEEP)
    num.partition(d, 1234).to_numpy()
    assert lib.b2s_launch_count(_lib.K_SWEEP) == before


def test_lexsort_long_keys_and_mixed_widths(cuda_device):
    """1-D keys long enough for the radix sort: the order so far rides through every key's passes."""
    rng = np.random.default_rng(9)
    n = 200_000
    keys = (rng.integers(0, 7, n).astype(np.int8), rng.standard_normal(n).astype(np.float32).round(1),
            rng.integers(0, 5, n).astype(np.uint64), rng.integers(0, 3, n).astype(np.float64),
            rng.integers(-2, 2, n).astype(np.int16))
    keys[1][::500] = np.nan
    keys[1][1::500] = -np.inf
    for take in (1, 2, 5):
        assert np.array_equal(num.lexsort(keys[:take]).to_numpy(), np.lexsort(keys[:take])), take
    # constant keys leave the order to the others; a single row of an N-D array; complex keys
    assert np.array_equal(num.lexsort((keys[0], np.zeros(n, np.int32))).to_numpy(), np.lexsort((keys[0], np.zeros(n, np.int32))))
    m1, m2 = rng.integers(0, 3, (3, 20_000)).astype(np.int32), rng.integers(0, 3, (3, 20_000)).astype(np.float32)
    assert np.array_equal(num.lexsort((m1, m2)).to_numpy(), np.lexsort((m1, m2)))
    c = (rng.integers(0, 3, 50_000) + 1j * rng.integers(0, 3, 50_000)).astype(np.complex128)
    assert np.array_equal(num.lexsort((keys[0][:50_000], c)).to_numpy(), np.lexsort((keys[0][:50_000], c)))
