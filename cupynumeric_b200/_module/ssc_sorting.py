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


# 1-D tiles longer than this take the selection kernels; shorter ones (and rows of N-D arrays,
# which the on-chip row sort handles at one read and one write) are simply sorted
SELECT_MIN = 8192


def _select_1d(a: ndarray, kth: Any, want_indices: bool):
    """Radix select + three-block partition of a 1-D array held by one process (``b2s_partition_1d``).
    Returns None when the case is not the selection's (several kth values, short or distributed array)."""
    import ctypes

    import torch

    from .. import _lib
    from ..runtime import runtime

    ks = np.atleast_1d(np.asarray(kth))
    if a.ndim != 1 or ks.size != 1 or a.size <= SELECT_MIN or runtime.num_procs > 1 or a.dtype == np.complex128:
        return None
    k = int(ks[0]) % a.size
    lib = _lib.lib()
    tile = a.torch().contiguous()
    out = torch.empty(tile.shape, dtype=torch.int64 if want_indices else tile.dtype, device=tile.device)
    need = ctypes.c_size_t()
    _lib.check(lib.b2s_partition_workspace_bytes(ctypes.byref(need)), "b2s_partition_workspace_bytes")
    ws = torch.empty(need.value, dtype=torch.uint8, device=tile.device)   # not the sorts' workspace: other contents
    st = lib.b2s_partition_1d(_lib.DTYPE_CODE[a.dtype], tile.data_ptr(), None if want_indices else out.data_ptr(),
                              out.data_ptr() if want_indices else None, tile.numel(), k, 0, ws.data_ptr(), ws.numel(),
                              runtime.stream_handle())
    _lib.check(st, "b2s_partition_1d")
    return array(out)


def partition(a: Any, kth: Any, axis: int | None = -1, kind: str = "introselect", order: Any = None) -> ndarray:
    """A partitioned copy of ``a``: the element of rank ``kth`` along ``axis`` is where a sort would
    put it, smaller elements come before it, larger ones after.  Long 1-D arrays go through a
    radix select (O(n) bytes); every other case is sorted along ``axis``, as the reference does for
    all of them ("falls back to sort for now", ``cupynumeric/_thunk/deferred.py:5476-5494``) - a
    sorted array satisfies the partition property for every ``kth``."""
    a = array(a)
    if order is not None:
        raise NotImplementedError(
            "cuPyNumeric does not support partitioning with 'order' as ndarray only supports numeric values")
    if axis is not None and a.ndim:
        if axis >= a.ndim or axis < -a.ndim:
            raise ValueError("invalid axis")
        _check_kth(kth, a.shape[axis])
    flat = a if axis is not None or a.ndim <= 1 else array(a.torch().reshape(-1))
    selected = _select_1d(flat, kth, False) if (axis is None or a.ndim == 1) else None
    return selected if selected is not None else sort(a, axis=axis)


def argpartition(a: Any, kth: Any, axis: int | None = -1, kind: str = "introselect", order: Any = None) -> ndarray:
    """Indices that partition ``a`` (see ``partition``); the full argsort where selection does not apply."""
    a = array(a)
    if order is not None:
        raise NotImplementedError(
            "cuPyNumeric does not support partitioning with 'order' as ndarray only supports numeric values")
    if axis is not None and a.ndim:
        if axis >= a.ndim or axis < -a.ndim:
            raise ValueError("invalid axis")
        _check_kth(kth, a.shape[axis])
    flat = a if axis is not None or a.ndim <= 1 else array(a.torch().reshape(-1))
    selected = _select_1d(flat, kth, True) if (axis is None or a.ndim == 1) else None
    return selected if selected is not None else argsort(a, axis=axis)


def lexsort(keys: Any, axis: int | None = -1) -> ndarray:
    """Stable lexicographic argsort over several keys, the last key being the most significant
    (``cupynumeric/_module/ssc_sorting.py:354-444``).  One call into the library
    (``b2s_lexsort``): a stable radix argsort per key with the order so far carried through it; the
    reference chains ARGSORT tasks and gathers from Python and first replaces NaN and infinities by
    finite stand-ins, which is not needed here because the sort itself orders
    -inf < finite < +inf < NaN.  Single process only."""
    import ctypes

    import torch

    from .. import _lib
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
    ndim = klist[0].ndim
    if axis >= ndim or axis < -ndim:
        raise ValueError("invalid axis")
    axis %= ndim
    # the sort axis last, dense (a no-op for the usual axis=-1 on contiguous keys)
    tiles = [k.torch().movedim(axis, -1).contiguous() for k in klist]
    shape = tiles[0].shape
    volume, segment = tiles[0].numel(), shape[-1]
    lib = _lib.lib()
    n = len(tiles)
    codes = (ctypes.c_int * n)(*[_lib.DTYPE_CODE[k.dtype] for k in klist])
    ptrs = (ctypes.c_void_p * n)(*[t.data_ptr() for t in tiles])
    need = ctypes.c_size_t()
    _lib.check(lib.b2s_lexsort_workspace_bytes(n, codes, volume, segment, ctypes.byref(need)), "b2s_lexsort_workspace_bytes")
    ws = torch.empty(max(need.value, 256), dtype=torch.uint8, device=tiles[0].device)
    out = torch.empty(shape, dtype=torch.int64, device=tiles[0].device)
    _lib.check(lib.b2s_lexsort(n, codes, ptrs, out.data_ptr(), volume, segment, ws.data_ptr(), ws.numel(),
                               runtime.stream_handle()), "b2s_lexsort")
    return array(out.movedim(-1, axis).contiguous() if axis != ndim - 1 else out)
