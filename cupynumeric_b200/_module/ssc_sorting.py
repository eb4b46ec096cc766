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
