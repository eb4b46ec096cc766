"""TEST INFRASTRUCTURE: NumPy restatement of the SORT task's result.

The reference's integration tests compare ``cupynumeric.sort/argsort`` with
``numpy.sort/argsort`` (``tests/integration/test_sort.py:85-102``,
``tests/integration/test_argsort.py:132-163``).  The task itself is always
stable on both of its back-ends (radix sort on GPU, merge sort on CPU), so the
expected result for every ``kind`` is NumPy's ``kind="stable"`` result.
"""
from __future__ import annotations

import numpy as np


def np_sort(a: np.ndarray, axis: int | None = -1) -> np.ndarray:
    """Expected output of ``cupynumeric.sort(a, axis)`` (``_module/ssc_sorting.py:77-121``)."""
    return np.sort(a, axis=axis, kind="stable")


def np_argsort(a: np.ndarray, axis: int | None = -1) -> np.ndarray:
    """Expected output of ``cupynumeric.argsort(a, axis, kind="stable")``; int64 indices
    (``_module/ssc_sorting.py:30-74``)."""
    return np.argsort(a, axis=axis, kind="stable").astype(np.int64, copy=False)


def np_task_sort(keys: np.ndarray, segment: int, argsort: bool, index_offset: int = 0,
                 ndim_is_1: bool = True) -> np.ndarray:
    """Expected output of ONE point task on a dense row-major tile.

    ``keys`` is the flattened tile, ``segment`` the extent of its last axis.  Index rule:
    1-D ``index_offset + i``; N-D ``i % segment + index_offset``
    (``src/cupynumeric/sort/sort.cu:1851-1862``, ``sort_cpu.inl:990-1002``).
    """
    keys = np.ascontiguousarray(keys).reshape(-1)
    if keys.size == 0:
        return np.empty(0, dtype=np.int64 if argsort else keys.dtype)
    rows = keys.reshape(-1, segment)
    if not argsort:
        return np.sort(rows, axis=-1, kind="stable").reshape(-1)
    idx = np.argsort(rows, axis=-1, kind="stable").astype(np.int64)
    if ndim_is_1:
        assert rows.shape[0] == 1
    return (idx + np.int64(index_offset)).reshape(-1)


def complex_lex_argsort(keys: np.ndarray, segment: int) -> np.ndarray:
    """Stable (real, imaginary) lexicographic argsort of every ``segment``-long row of a complex
    tile, with NaN last inside each part and -0.0 == +0.0; positions inside the row.

    The reference compares complex keys with raw ``<`` on the parts
    (``src/cupynumeric/binary/binary_op_util.h:32-36``), which leaves the place of NaN parts open
    and is this order for NaN-free input.  For NaN-free input it is also NumPy's order, which is
    what the reference's tests check (parity unpinned for NaN parts: NumPy puts every key with a
    NaN imaginary part after all keys without one, whatever the real parts)."""
    keys = np.ascontiguousarray(keys).reshape(-1)
    out = np.empty(keys.size, dtype=np.int64)
    for s0 in range(0, keys.size, segment):
        c = keys[s0:s0 + segment]
        re, im = c.real, c.imag
        out[s0:s0 + segment] = np.lexsort((np.nan_to_num(im, nan=0.0), np.isnan(im),
                                           np.nan_to_num(re, nan=0.0), np.isnan(re)))
    return out
