"""``sort`` and ``argsort``: the module-level entry points of the SORT path, with the
signatures and result conventions of ``cupynumeric/_module/ssc_sorting.py:30-121``."""
from __future__ import annotations

from typing import Any

import numpy as np

from .._array import array, ndarray


def argsort(a: Any, axis: int | None = -1, kind: str = "quicksort", order: Any = None) -> ndarray:
    """Indices that would sort ``a`` along ``axis`` (flattened when ``axis`` is None); int64.

    ``kind``: 'quicksort', 'mergesort', 'heapsort' or 'stable'; the result is stable for all of
    them.  ``order`` is not supported."""
    a = array(a)
    result = ndarray((a.size,) if axis is None else a.shape, np.int64)
    result._thunk.sort(rhs=a._thunk, argsort=True, axis=axis, kind=kind, order=order)
    return result


def sort(a: Any, axis: int | None = -1, kind: str = "quicksort", order: Any = None) -> ndarray:
    """A sorted copy of ``a`` along ``axis`` (flattened when ``axis`` is None)."""
    a = array(a)
    result = ndarray((a.size,) if axis is None else a.shape, a.dtype)
    result._thunk.sort(rhs=a._thunk, axis=axis, kind=kind, order=order)
    return result


def searchsorted(a: Any, v: Any, side: str = "left", sorter: Any = None) -> ndarray:
    """Indices where the elements of ``v`` should be inserted into the sorted 1-D array ``a`` to
    keep it sorted.  Same checks and type promotion as ``ndarray.searchsorted``
    (``cupynumeric/_array/array.py:3702-3771``): ``a`` must be 1-D; ``a`` and ``v`` are brought to
    their common dtype; ``sorter``, if given, is applied with a gather first."""
    from .._thunk.deferred import DeferredArray, to_torch_dtype

    a = array(a)
    if a.ndim != 1:
        raise ValueError("Dimension mismatch: self must be a 1D array")
    if side not in ("left", "right"):
        raise ValueError("side must be 'left' or 'right'")
    v = array(np.asarray(v) if not hasattr(v, "_thunk") and not hasattr(v, "is_cuda") else v)
    a_t, v_t = a._thunk, v._thunk
    if a.dtype != v.dtype:
        common = np.result_type(a.dtype, v.dtype)
        if v.dtype != common:
            v_t = DeferredArray(v_t.base.to(to_torch_dtype(common)), global_lo=v_t.global_lo)
        if a.dtype != common:
            a_t = DeferredArray(a_t.base.to(to_torch_dtype(common)), global_lo=a_t.global_lo)
    if sorter is not None and a.shape[0] > 1:
        sorter = array(sorter)
        if sorter.ndim != 1:
            raise ValueError("Dimension mismatch: sorter must be a 1D array")
        if sorter.shape != a.shape:
            raise ValueError("Shape mismatch: sorter must have the same shape as self")
        if not np.issubdtype(sorter.dtype, np.integer):
            raise ValueError("Dtype mismatch: sorter must be of integer type")
        a_t = DeferredArray(a_t.base[sorter.torch().long()].contiguous(), global_lo=a_t.global_lo)
    result = ndarray(v.shape, np.int64)
    result._thunk.searchsorted(a_t, v_t, side)
    return result


def sort_complex(a: Any) -> ndarray:
    """Sorts with the real part first, the imaginary part second, and returns a complex array
    (``cupynumeric/_module/ssc_sorting.py:124-157``): complex input keeps its dtype, integers of
    at most 16 bits become complex64, everything else complex128."""
    import torch

    result = sort(a)
    if np.issubdtype(result.dtype, np.complexfloating):
        return result
    small_int = np.issubdtype(result.dtype, np.integer) and result.dtype.itemsize <= 2
    return array(result.torch().to(torch.complex64 if small_int else torch.complex128))


def _check_kth(kth: Any, extent: int) -> None:
    for k in np.atleast_1d(np.asarray(kth)).tolist():
        if not -extent <= int(k) < extent:
            raise ValueError(f"kth(={k}) out of bounds ({extent})")


def partition(a: Any, kth: Any, axis: int | None = -1, kind: str = "introselect", order: Any = None) -> ndarray:
    """A partitioned copy of ``a``.  Like the reference, which "falls back to sort for now"
    (``cupynumeric/_thunk/deferred.py:5476-5494``), the result is fully sorted along ``axis``,
    which satisfies the partition property for every ``kth``."""
    a = array(a)
    if order is not None:
        raise NotImplementedError(
            "cuPyNumeric does not support partitioning with 'order' as ndarray only supports numeric values")
    if axis is not None and a.ndim:
        if axis >= a.ndim or axis < -a.ndim:
            raise ValueError("invalid axis")
        _check_kth(kth, a.shape[axis])
    return sort(a, axis=axis)


def argpartition(a: Any, kth: Any, axis: int | None = -1, kind: str = "introselect", order: Any = None) -> ndarray:
    """Indices that partition ``a``; the full argsort, as in the reference."""
    a = array(a)
    if order is not None:
        raise NotImplementedError(
            "cuPyNumeric does not support partitioning with 'order' as ndarray only supports numeric values")
    if axis is not None and a.ndim:
        if axis >= a.ndim or axis < -a.ndim:
            raise ValueError("invalid axis")
        _check_kth(kth, a.shape[axis])
    return argsort(a, axis=axis)


def lexsort(keys: Any, axis: int | None = -1) -> ndarray:
    """Stable lexicographic argsort over several keys, the last key being the most significant:
    one stable argsort per key, each applied to the key reordered by the indices so far
    (``cupynumeric/_module/ssc_sorting.py:423-444``).  The reference first replaces NaN and
    infinities by finite stand-ins (``:354-421``); that is not needed here because the sort
    itself orders -inf < finite < +inf < NaN.  Single process only."""
    import torch

    from ..runtime import runtime

    if keys is None:
        raise TypeError("'NoneType' object is not iterable")
    if axis is None:
        raise TypeError("'NoneType' object cannot be interpreted as an integer")
    if runtime.num_procs > 1:
        raise NotImplementedError("lexsort over tiles held by several processes")
    klist = [array(k) for k in keys]
    if len(klist) == 0:
        raise TypeError("Need at least one key to sort")
    first_shape = klist[0].shape
    for i, key in enumerate(klist[1:], 1):
        if key.shape != first_shape:
            raise ValueError(
                f"All keys must have the same shape. Key {i} has shape {key.shape}, expected {first_shape}")
    if klist[0].ndim == 0:
        return array(np.zeros((), dtype=np.int64))
    if klist[0].size == 0:
        return array(np.empty(first_shape, dtype=np.int64))
    indices = argsort(klist[0], axis=axis, kind="stable").torch()
    for key in klist[1:]:
        reordered = torch.take_along_dim(key.torch(), indices, dim=axis)
        order = argsort(array(reordered), axis=axis, kind="stable").torch()
        indices = torch.take_along_dim(indices, order, dim=axis)
    return array(indices)
