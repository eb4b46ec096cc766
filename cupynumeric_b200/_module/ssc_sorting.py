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
