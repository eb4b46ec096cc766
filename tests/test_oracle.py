"""Pins the CPU oracle: against the golden vectors of the reference's own C++ tests, against
NumPy's stable sort (the oracle of the reference's Python tests), and the two restatements
against each other."""
import json
import os

import numpy as np
import pytest

from oracle import complex_lex_argsort, np_argsort, np_sort, np_task_sort, thrust_task_sort

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")
SORT = json.load(open(os.path.join(GOLDEN, "sort_cc.json")))
ARGSORT = json.load(open(os.path.join(GOLDEN, "argsort_cc.json")))


def as_array(values, dtype):
    if dtype == "complex64":
        return np.array([complex(r, i) for r, i in values], dtype=np.complex64)
    return np.array(values, dtype=dtype)


def task_sort_along_axis(a: np.ndarray, axis: int, argsort: bool, backend: str):
    """Applies the point task the way the dispatch does: sort axis moved last, dense copy."""
    moved = np.ascontiguousarray(np.swapaxes(a, axis, -1))
    keys, idx = thrust_task_sort(moved, moved.shape[-1], argsort, ndim_is_1=(a.ndim == 1), backend=backend)
    out = (idx if argsort else keys).reshape(moved.shape)
    return np.swapaxes(out, -1, axis)


def golden_sort_cases():
    for dtype in ("int32", "float64", "complex64"):
        for shape, table in zip(SORT["shapes"], SORT[dtype]["expect"]):
            for axis, expect in table.items():
                yield dtype, tuple(shape), int(axis), expect


@pytest.mark.parametrize("dtype,shape,axis,expect", list(golden_sort_cases()))
def test_oracles_reproduce_reference_sort_tables(dtype, shape, axis, expect):
    a = as_array(SORT[dtype]["input"], dtype).reshape(shape)
    want = as_array(expect, dtype).reshape(shape)
    assert np.array_equal(np_sort(a, axis), want)
    for backend in ("host", "omp"):
        assert np.array_equal(task_sort_along_axis(a, axis, False, backend), want)


def golden_argsort_cases():
    for group in ("basic", "stable"):
        for dtype in ("int32", "float64", "complex64"):
            for shape, table in zip(ARGSORT["shapes"], ARGSORT["expect"]):
                for axis, expect in table.items():
                    yield group, dtype, tuple(shape), int(axis), expect
    for case in ARGSORT["maxdim"]["cases"]:
        for shape, table in zip(case["shapes"], case["expect"]):
            for axis, expect in table.items():
                yield "maxdim", "int32", tuple(shape), int(axis), expect


@pytest.mark.parametrize("group,dtype,shape,axis,expect", list(golden_argsort_cases()))
def test_oracles_reproduce_reference_argsort_tables(group, dtype, shape, axis, expect):
    src = ARGSORT["maxdim"]["input"] if group == "maxdim" else ARGSORT[group][dtype]
    a = as_array(src, dtype).reshape(shape)
    want = np.array(expect, dtype=np.int64).reshape(shape)
    assert np.array_equal(np_argsort(a, axis), want)
    for backend in ("host", "omp"):
        assert np.array_equal(task_sort_along_axis(a, axis, True, backend), want)


def test_oracles_reproduce_reference_large_descending_case():
    count = ARGSORT["large"]["count"]
    want = np.arange(count - 1, -1, -1, dtype=np.int64)
    for a in (np.arange(count, 0, -1, dtype=np.int32),
              (count * 1.1 - np.arange(count)).astype(np.float64)):
        assert np.array_equal(np_argsort(a), want)
        _, idx = thrust_task_sort(a, count, True)
        assert np.array_equal(idx, want)


@pytest.mark.parametrize("shape", [tuple(s) for s in SORT["empty_shapes"] + SORT["single_shapes"]])
def test_oracle_empty_and_single(shape):
    a = np.full(shape, 12, dtype=np.int32)
    for axis in range(-len(shape) + 1, len(shape)):
        assert np.array_equal(np_sort(a, axis), a)
        assert np.array_equal(np_argsort(a, axis), np.zeros(shape, dtype=np.int64))


DTYPES = [np.bool_, np.int8, np.int16, np.int32, np.int64, np.uint8, np.uint16, np.uint32, np.uint64,
          np.float16, np.float32, np.float64]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("backend", ["host", "omp"])
def test_thrust_oracle_equals_numpy_stable(dtype, backend):
    rng = np.random.default_rng(7)
    a = rng.integers(-100, 100, 6000)
    a = (np.abs(a) if np.dtype(dtype).kind in "ub" else a).astype(dtype)
    for segment in (6000, 100):
        for argsort in (False, True):
            keys, idx = thrust_task_sort(a, segment, argsort, index_offset=5, ndim_is_1=segment == 6000,
                                         backend=backend)
            want = np_task_sort(a, segment, argsort, index_offset=5, ndim_is_1=segment == 6000)
            assert np.array_equal(idx if argsort else keys, want)


def test_nan_last_contract_and_literal_reference_behaviour():
    rng = np.random.default_rng(11)
    a = rng.standard_normal(1 << 14).astype(np.float32)
    a[rng.choice(a.size, a.size // 100, replace=False)] = np.nan
    a[:4] = [0.0, -0.0, 0.0, -0.0]
    keys, idx = thrust_task_sort(a, a.size, True)  # NaN-last comparator is picked automatically
    assert np.array_equal(idx, np.argsort(a, kind="stable"))
    assert np.array_equal(keys.view(np.uint32), a[idx].view(np.uint32))
    n_nan = int(np.isnan(a).sum())
    assert np.isnan(keys[-n_nan:]).all() and not np.isnan(keys[:-n_nan]).any()
    # NaN-free: the literal reference comparator and the NaN-last one agree bit for bit
    b = a[~np.isnan(a)]
    k0, i0 = thrust_task_sort(b, b.size, True, nan_mode="literal")
    k1, i1 = thrust_task_sort(b, b.size, True, nan_mode="nan_last")
    assert np.array_equal(i0, i1) and np.array_equal(k0.view(np.uint32), k1.view(np.uint32))


def test_index_rules():
    a = np.array([3, 1, 2, 9, 8, 7], dtype=np.int32)
    _, idx = thrust_task_sort(a, 6, True, index_offset=100, ndim_is_1=True)
    assert idx.tolist() == [101, 102, 100, 105, 104, 103]
    _, idx = thrust_task_sort(a, 3, True, index_offset=10, ndim_is_1=False)
    assert idx.tolist() == [11, 12, 10, 12, 11, 10]


@pytest.mark.parametrize("dtype", [np.complex64, np.complex128])
def test_complex_order_contract(dtype):
    """Without NaN parts the documented complex order is NumPy's (and the golden tables');
    with NaN parts it is lexicographic with NaN last inside each part."""
    rng = np.random.default_rng(9)
    a = (rng.integers(-8, 8, 6 * 500) + 1j * rng.integers(-8, 8, 6 * 500)).astype(dtype)
    a.real[::11] = -0.0
    assert np.array_equal(complex_lex_argsort(a, 500), np_task_sort(a, 500, True, ndim_is_1=False))
    nan = np.nan
    b = np.array([complex(1, nan), complex(2, 0), complex(nan, 1), complex(1, 5), complex(nan, nan), complex(nan, -1),
                  complex(-np.inf, nan), complex(1, -np.inf)], dtype=dtype)
    assert complex_lex_argsort(b, b.size).tolist() == [6, 7, 3, 0, 1, 5, 2, 4]
