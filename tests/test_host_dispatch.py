"""Host-side dispatch (axis routing, error behaviour, tile bookkeeping) on CPU: the point-task
body is replaced by an oracle-backed stand-in, so only the Python layer that mirrors
``cupynumeric/_thunk/_sort.py`` and ``DeferredArray.sort`` is under test."""
import numpy as np
import pytest
import torch
from numpy.exceptions import AxisError

from cupynumeric_b200._thunk import _sort as sort_mod
from cupynumeric_b200._thunk.deferred import DeferredArray, create_deferred_thunk, to_torch_dtype
from oracle import np_argsort, np_sort, np_task_sort


@pytest.fixture()
def cpu_point_task(monkeypatch):
    """Stand-in for the CUDA point task: same contract as ``local_sort_tile``."""
    calls = []

    def fake(tile, argsort, stable, index_offset=0, out=None):
        assert tile.is_contiguous()
        a = tile.numpy()
        seg = a.shape[-1] if a.ndim else 1
        res = np_task_sort(a, max(seg, 1), argsort, index_offset=index_offset, ndim_is_1=a.ndim == 1)
        calls.append((tuple(a.shape), argsort, stable, index_offset))
        return torch.from_numpy(np.ascontiguousarray(res.reshape(a.shape)))

    monkeypatch.setattr(sort_mod, "local_sort_tile", fake)
    return calls


def run(a, argsort, axis, kind="quicksort"):
    rhs = DeferredArray(torch.from_numpy(a.copy()))
    shape = (a.size,) if axis is None else a.shape
    out = create_deferred_thunk(shape, np.int64 if argsort else a.dtype)
    out.sort(rhs, argsort=argsort, axis=axis, kind=kind)
    return out.base.numpy()


SHAPES = [(1,), (5,), (1, 5), (5, 1), (3, 4), (2, 3, 4), (4, 1, 3), (0,), (0, 3), (3, 0), (2, 2, 1, 4)]


@pytest.mark.parametrize("shape", SHAPES)
def test_routing_all_axes(cpu_point_task, shape):
    rng = np.random.default_rng(1)
    a = rng.integers(-50, 50, shape).astype(np.int32)
    for axis in [None] + list(range(-len(shape), len(shape))):
        assert np.array_equal(run(a, False, axis), np_sort(a, axis)), (shape, axis)
        assert np.array_equal(run(a, True, axis, kind="stable"), np_argsort(a, axis)), (shape, axis)


def test_only_kind_stable_sets_the_flag(cpu_point_task):
    a = np.arange(6, dtype=np.int32)
    for kind, want in (("quicksort", False), ("mergesort", False), ("heapsort", False), ("stable", True)):
        cpu_point_task.clear()
        run(a, False, -1, kind)
        assert cpu_point_task[-1][2] is want


def test_swapped_axis_sorts_a_dense_copy_of_the_last_axis(cpu_point_task):
    a = np.random.default_rng(2).integers(0, 9, (3, 4, 5)).astype(np.int32)
    run(a, False, 0)
    assert cpu_point_task[-1][0] == (5, 4, 3)      # axis 0 swapped to the end
    run(a, False, None)
    assert cpu_point_task[-1][0] == (60,)          # flattened


def test_error_behaviour_matches_the_reference():
    a = DeferredArray(torch.zeros((2, 3), dtype=torch.int32))
    out = create_deferred_thunk((2, 3), np.int32)
    for bad in (2, -3):
        with pytest.raises(ValueError, match="invalid axis"):
            out.sort(a, axis=bad)
    with pytest.raises(NotImplementedError):
        out.sort(a, order="x")
    scalar = DeferredArray(torch.zeros((), dtype=torch.int32))
    with pytest.raises(AxisError):
        sort_mod.sort_deferred(create_deferred_thunk((), np.int32), scalar, False, axis=0)
    sort_mod.sort_deferred(out, scalar, False, axis=None)  # 0-D with axis=None: returned as is
    assert out.base.ndim == 0
    with pytest.raises(TypeError):
        to_torch_dtype(np.dtype("U4"))


def test_one_dim_tiles_carry_their_global_offset(cpu_point_task):
    a = np.array([5, 1, 4], dtype=np.int64)
    rhs = DeferredArray(torch.from_numpy(a), global_lo=100)
    out = create_deferred_thunk((3,), np.int64)
    out.sort(rhs, argsort=True, axis=0, kind="stable")
    assert out.base.tolist() == [101, 102, 100] and cpu_point_task[-1][3] == 100
