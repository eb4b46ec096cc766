"""GPU parity: the CUDA path, called through the C ABI, against the CPU oracle on the same
seeded inputs - bit-exact keys, identical indices."""
import json
import os

import numpy as np
import pytest

from oracle import complex_lex_argsort, np_argsort, np_sort, np_task_sort, thrust_task_sort
from tests.helpers import ALL_DTYPES, assert_bit_equal, cabi_local_sort, random_keys, to_device, to_host

pytestmark = pytest.mark.gpu

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def expected(keys, segment, argsort, index_offset=0, ndim_is_1=True):
    """Oracle result for one tile: (sorted keys, indices)."""
    k, i = thrust_task_sort(keys, segment, True, index_offset=index_offset, ndim_is_1=ndim_is_1)
    return k, i


# ---- 1-D, every dtype, sizes around the tile boundaries of both kernels -----------------------
SIZES_1D = [1, 2, 31, 32, 33, 127, 128, 129, 1000, 4095, 4096, 4097, 8191, 8192, 8193, 8192 * 3 + 5,
            100_000, (1 << 20) + 3]


@pytest.mark.parametrize("dtype", ALL_DTYPES)
@pytest.mark.parametrize("flavour", ["full", "small"])
def test_sort_and_argsort_1d_all_sizes(cuda_device, dtype, flavour):
    rng = np.random.default_rng(1234)
    for n in SIZES_1D:
        a = random_keys(rng, dtype, n, flavour)
        want_k, want_i = expected(a, n, True, index_offset=7)
        got_k, _ = cabi_local_sort(a, n, False)
        assert_bit_equal(got_k, want_k, f"sort {np.dtype(dtype)} n={n}")
        _, got_i = cabi_local_sort(a, n, True, index_offset=7)
        assert np.array_equal(got_i, want_i), f"argsort {np.dtype(dtype)} n={n}"


@pytest.mark.parametrize("dtype", [np.uint8, np.int16, np.float16, np.int32, np.float32, np.int64, np.float64])
def test_more_tiles_than_the_gpu_holds_at_once(cuda_device, dtype):
    """2^23 + 5 keys per key width: over a thousand tiles per pass, several waves of CTAs, so the
    chained look-back crosses CTAs that are not resident together; the histogram kernel with a
    copy of the tables per lane runs here too.  Bit for bit against the oracle."""
    rng = np.random.default_rng(2323)
    n = (1 << 23) + 5
    a = random_keys(rng, dtype, n, "full")
    want_k, want_i = expected(a, n, True, index_offset=3)
    got_k, _ = cabi_local_sort(a, n, False)
    assert_bit_equal(got_k, want_k, f"sort {np.dtype(dtype)}")
    _, got_i = cabi_local_sort(a, n, True, index_offset=3)
    assert np.array_equal(got_i, want_i), f"argsort {np.dtype(dtype)}"


@pytest.mark.parametrize("dtype", [np.int32, np.float32, np.uint64, np.float64, np.int8, np.float16])
def test_inplace_and_keys_with_indices(cuda_device, dtype):
    rng = np.random.default_rng(99)
    for n in (5000, 50_000, 300_000):
        a = random_keys(rng, dtype, n, "small")
        want_k, want_i = expected(a, n, True)
        got_k, _ = cabi_local_sort(a, n, False, inplace=True)
        assert_bit_equal(got_k, want_k, "in place")
        got_k, got_i = cabi_local_sort(a, n, True, want_keys_too=True)
        assert_bit_equal(got_k, want_k, "keys beside indices")
        assert np.array_equal(got_i, want_i)


@pytest.mark.parametrize("dtype", [np.int32, np.int64, np.float32, np.uint8])
def test_constant_and_presorted_inputs_skip_passes(cuda_device, dtype):
    """All-equal keys (every pass is skipped), one varying byte (one pass, also in place),
    ascending and descending runs."""
    n = 70_000
    cases = [np.full(n, 5, dtype=dtype), (np.arange(n) % 200).astype(dtype),
             np.arange(n).astype(dtype), np.arange(n, 0, -1).astype(dtype)]
    for a in cases:
        want_k, want_i = expected(a, n, True)
        got_k, _ = cabi_local_sort(a, n, False)
        assert_bit_equal(got_k, want_k)
        got_k, _ = cabi_local_sort(a, n, False, inplace=True)
        assert_bit_equal(got_k, want_k)
        _, got_i = cabi_local_sort(a, n, True)
        assert np.array_equal(got_i, want_i)


def test_chunked_path_above_the_single_sort_limit(cuda_device, monkeypatch):
    """1-D tiles at or above the single-sort limit are sorted in chunks and merged; the limit is
    lowered here so that a small array takes that path."""
    monkeypatch.setenv("B2S_MAX_1D_LOG2", "16")
    rng = np.random.default_rng(31)
    for dtype, n in ((np.int32, 300_001), (np.float32, 65_536), (np.uint64, 1_000_000), (np.int8, 70_000)):
        a = random_keys(rng, dtype, n, "small" if dtype == np.uint64 else "full")
        want_k, want_i = expected(a, n, True, index_offset=9)
        got_k, got_i = cabi_local_sort(a, n, True, index_offset=9, want_keys_too=True)
        assert np.array_equal(got_i, want_i), np.dtype(dtype)
        assert_bit_equal(got_k, want_k)
        got_k, _ = cabi_local_sort(a, n, False, inplace=True)
        assert_bit_equal(got_k, want_k)


def test_one_dim_tile_beyond_two_to_the_thirty(cuda_device):
    """2^30 + 12345 uint8 keys in one tile (chunks of 2^29 + merge).  The expected output follows
    from the histogram alone: value v repeated count[v] times."""
    n = (1 << 30) + 12345
    rng = np.random.default_rng(5)
    a = rng.integers(0, 256, n, dtype=np.uint8)
    got, _ = cabi_local_sort(a, n, False)
    counts = np.bincount(a, minlength=256)
    assert np.array_equal(np.bincount(got, minlength=256), counts)
    assert bool(np.all(got[1:] >= got[:-1]))


# ---- segmented (axis sorts) --------------------------------------------------------------------
SEGMENTS = [(7, 1), (5, 2), (1000, 3), (64, 12), (33, 128), (20, 129), (9, 1000), (5, 1024), (3, 1025),
            (4, 4096), (3, 4097), (2, 8192), (3, 8193), (2, 20000), (37, 8200), (6, 50001)]


@pytest.mark.parametrize("dtype", ALL_DTYPES)
def test_segmented_sort_and_argsort(cuda_device, dtype):
    rng = np.random.default_rng(4321)
    for nseg, seg in SEGMENTS:
        a = random_keys(rng, dtype, nseg * seg, "small" if seg % 2 else "full")
        want_k, want_i = expected(a, seg, True, index_offset=3, ndim_is_1=False)
        got_k, _ = cabi_local_sort(a, seg, False, ndim_is_1=False)
        assert_bit_equal(got_k, want_k, f"segsort {np.dtype(dtype)} {nseg}x{seg}")
        _, got_i = cabi_local_sort(a, seg, True, index_offset=3, ndim_is_1=False)
        assert np.array_equal(got_i, want_i), f"segargsort {np.dtype(dtype)} {nseg}x{seg}"


def test_float_special_values(cuda_device):
    """NaNs of both signs and several payloads last and in input order; -0.0 and +0.0 tie."""
    for dt, u in ((np.float32, np.uint32), (np.float64, np.uint64), (np.float16, np.uint16)):
        fi = np.finfo(dt)
        nbits = np.dtype(dt).itemsize * 8
        qnan = np.array([np.nan], dtype=dt).view(u)[0]
        neg_nan = u(qnan | (u(1) << u(nbits - 1)))
        pay_nan = u(qnan | u(5))
        specials = np.array([0.0, -0.0, np.inf, -np.inf, fi.max, fi.min, fi.tiny, -fi.tiny,
                             fi.smallest_subnormal, -fi.smallest_subnormal, 1.0, -1.0], dtype=dt)
        raw = np.concatenate([specials.view(u), np.array([qnan, neg_nan, pay_nan], dtype=u)])
        rng = np.random.default_rng(5)
        a = raw[rng.integers(0, raw.size, 30_000)].view(dt)
        for seg in (a.size, 100):
            want_k, want_i = expected(a, seg, True, ndim_is_1=seg == a.size)
            assert np.array_equal(want_i.reshape(-1, seg),
                                  np.argsort(a.reshape(-1, seg), axis=-1, kind="stable"))
            got_k, got_i = cabi_local_sort(a, seg, True, ndim_is_1=seg == a.size, want_keys_too=True)
            assert np.array_equal(got_i, want_i)
            assert_bit_equal(got_k, want_k)


# ---- the reference's own golden vectors through the public API ---------------------------------
def test_reference_golden_vectors_through_api(cuda_device):
    import cupynumeric_b200 as num

    sort_g = json.load(open(os.path.join(GOLDEN, "sort_cc.json")))
    arg_g = json.load(open(os.path.join(GOLDEN, "argsort_cc.json")))
    def arr(values, dtype):
        if dtype == "complex64":
            return np.array([complex(r, i) for r, i in values], dtype=np.complex64)
        return np.array(values, dtype=dtype)

    for dtype in ("int32", "float64", "complex64"):
        for shape, table in zip(sort_g["shapes"], sort_g[dtype]["expect"]):
            a = arr(sort_g[dtype]["input"], dtype).reshape(shape)
            for axis, expect in table.items():
                for kind in ("quicksort", "mergesort", "heapsort", "stable"):
                    got = num.sort(a, axis=int(axis), kind=kind).to_numpy()
                    assert np.array_equal(got, arr(expect, dtype).reshape(shape)), (shape, axis)
        for group in ("basic", "stable"):
            for shape, table in zip(arg_g["shapes"], arg_g["expect"]):
                a = arr(arg_g[group][dtype], dtype).reshape(shape)
                for axis, expect in table.items():
                    got = num.argsort(a, axis=int(axis), kind="stable").to_numpy()
                    assert np.array_equal(got, np.array(expect, dtype=np.int64).reshape(shape))
    for case in arg_g["maxdim"]["cases"]:
        for shape, table in zip(case["shapes"], case["expect"]):
            a = np.array(arg_g["maxdim"]["input"], dtype=np.int32).reshape(shape)
            for axis, expect in table.items():
                got = num.argsort(a, axis=int(axis)).to_numpy()
                assert np.array_equal(got, np.array(expect, dtype=np.int64).reshape(shape))
    count = arg_g["large"]["count"]
    for a in (np.arange(count, 0, -1, dtype=np.int32), (count * 1.1 - np.arange(count)).astype(np.float64)):
        assert np.array_equal(num.argsort(a).to_numpy(), np.arange(count - 1, -1, -1))
    for shape in sort_g["empty_shapes"] + sort_g["single_shapes"]:
        a = np.full(shape, 12, dtype=np.int32)
        for axis in range(-len(shape) + 1, len(shape)):
            assert np.array_equal(num.sort(a, axis=axis).to_numpy(), a)
            assert np.array_equal(num.argsort(a, axis=axis).to_numpy(), np.zeros(shape, dtype=np.int64))


@pytest.mark.parametrize("dtype", [np.complex64, np.complex128])
def test_complex_lexicographic_order(cuda_device, dtype):
    """(real, imag) lexicographic, stable; many ties in the real parts."""
    rng = np.random.default_rng(77)
    for n, seg in ((1, 1), (1000, 1000), (70_000, 70_000), (64 * 300, 300), (5 * 9000, 9000)):
        a = (rng.integers(-20, 20, n) + 1j * rng.integers(-20, 20, n)).astype(dtype)
        want_k, want_i = expected(a, seg, True, index_offset=5, ndim_is_1=seg == n)
        got_k, got_i = cabi_local_sort(a, seg, True, index_offset=5, ndim_is_1=seg == n, want_keys_too=True)
        assert np.array_equal(got_i, want_i), (n, seg)
        assert np.array_equal(got_k, want_k)
        got_k, _ = cabi_local_sort(a, seg, False, ndim_is_1=seg == n, inplace=True)
        assert np.array_equal(got_k, want_k)


@pytest.mark.parametrize("dtype", [np.complex64, np.complex128])
def test_complex_special_values(cuda_device, dtype):
    rng = np.random.default_rng(78)
    pool = np.array([0.0, -0.0, 1.5, -1.5, np.inf, -np.inf, np.nan, 1e-40, -1e-40, 3.0])
    for n, seg in ((4000, 4000), (50_000, 50_000), (40 * 500, 500), (3 * 10_000, 10_000)):
        a = (rng.choice(pool, n) + 1j * rng.choice(pool, n)).astype(dtype)
        a.real[rng.integers(0, n, n // 7)] = -0.0     # signed zeros in both parts
        order = complex_lex_argsort(a, seg)
        want_k = a.reshape(-1, seg)[np.arange(n // seg)[:, None], order.reshape(-1, seg)].reshape(-1)
        got_k, got_i = cabi_local_sort(a, seg, True, index_offset=0, ndim_is_1=seg == n, want_keys_too=True)
        assert np.array_equal(got_i, order), (n, seg)
        assert np.array_equal(got_k.view(np.uint8), want_k.view(np.uint8))


# ---- the reference's Python test shapes (tests/integration/test_sort.py:21-40) -----------------
REF_PY_SHAPES = [(1,), (5,), (1, 5), (5, 1), (3, 3), (1, 1, 5), (5, 1, 1), (3, 3, 3), (2, 3, 4),
                 (0,), (0, 3), (3, 0), (2, 0, 3), (4, 5, 6), (7, 1, 3), (1, 1, 1), (6, 6)]


def test_api_all_axes_small_shapes(cuda_device):
    import cupynumeric_b200 as num

    rng = np.random.default_rng(42)
    for shape in REF_PY_SHAPES:
        a = rng.integers(-100, 100, shape).astype(np.int32)
        for axis in [None] + list(range(-len(shape), len(shape))):
            assert np.array_equal(num.sort(a, axis=axis).to_numpy(), np_sort(a, axis)), (shape, axis)
            assert np.array_equal(num.argsort(a, axis=axis, kind="stable").to_numpy(), np_argsort(a, axis))
    b = rng.integers(-100, 100, (4, 5, 6)).astype(np.int32)
    arr = num.array(b)
    arr.sort(axis=1)
    assert np.array_equal(arr.to_numpy(), np.sort(b, axis=1))


# ---- reduced-size versions of the benchmark configurations --------------------------------------
def test_config_shapes_reduced(cuda_device):
    from cupynumeric_b200 import workloads as w

    a = w.c1_int32_uniform(1 << 20)
    got, _ = cabi_local_sort(a, a.size, False)
    assert_bit_equal(got, np.sort(a, kind="stable"))

    a = w.c2_float32_nan_dups(1 << 21)
    _, got = cabi_local_sort(a, a.size, True)
    assert np.array_equal(got, np.argsort(a, kind="stable"))

    a = w.c3_float64_rows((512, 4096))
    got, _ = cabi_local_sort(a, 4096, False, ndim_is_1=False)
    assert_bit_equal(got.reshape(a.shape), np.sort(a, axis=-1, kind="stable"))

    a = w.c4_int64_zipf_shard(1 << 20)
    got, _ = cabi_local_sort(a, a.size, False)
    assert_bit_equal(got, np.sort(a, kind="stable"))

    a = w.c5_uint64_nearly_sorted_shard(1 << 20)
    _, got = cabi_local_sort(a, a.size, True)
    assert np.array_equal(got, np.argsort(a, kind="stable"))


def test_bounded_wait_runs_out_and_is_reported(cuda_device):
    """A look-back wait that can never be satisfied (the library's own self-test: the first tile of
    a small sort is never processed) ends after a few thousand polls: the kernels return, the
    status word reads B2S_ERR_TIMEOUT, and the same workspace then serves a correct sort."""
    import ctypes

    import torch

    from cupynumeric_b200 import _lib

    lib = _lib.lib()
    ws = torch.empty(8 << 20, dtype=torch.uint8, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    assert lib.b2s_selftest_wait_timeout(ws.data_ptr(), ws.numel(), stream) == 0
    assert lib.b2s_check_status(ws.data_ptr(), stream) == 5          # B2S_ERR_TIMEOUT
    a = np.random.default_rng(0).integers(0, 1 << 31, 100_000).astype(np.uint32)
    d_in, d_out = to_device(a), torch.empty(a.size, dtype=torch.int32, device="cuda")
    need = ctypes.c_size_t()
    _lib.check(lib.b2s_workspace_bytes(_lib.DTYPE_CODE[a.dtype], a.size, a.size, 0, ctypes.byref(need)), "ws")
    assert need.value <= ws.numel()
    _lib.check(lib.b2s_local_sort(_lib.DTYPE_CODE[a.dtype], d_in.data_ptr(), d_out.data_ptr(), None, a.size, a.size, 0, 1, 1,
                                  ws.data_ptr(), ws.numel(), stream), "b2s_local_sort")
    assert lib.b2s_check_status(ws.data_ptr(), stream) == 0
    assert np.array_equal(to_host(d_out, a.dtype), np.sort(a))
