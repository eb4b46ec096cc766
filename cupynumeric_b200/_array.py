"""``ndarray``: the minimal array object the sort API needs (construction from host or device
memory, shape/dtype, ``sort``/``argsort`` methods, conversion back to NumPy).  Stands for the
sort-related surface of ``cupynumeric/_array/array.py`` (``sort`` ``:3774-3796``, ``argsort``
``:3798-3825``)."""
from __future__ import annotations

from typing import Any

import numpy as np
import torch

from ._thunk.deferred import DeferredArray, create_deferred_thunk, to_torch_dtype
from .runtime import runtime


class ndarray:
    def __init__(self, shape: tuple[int, ...], dtype: Any, thunk: DeferredArray | None = None) -> None:
        to_torch_dtype(dtype)  # TypeError for dtypes the task cannot take (strings, objects, ...)
        self._thunk = thunk if thunk is not None else create_deferred_thunk(tuple(shape), dtype)

    @property
    def shape(self) -> tuple[int, ...]:
        return self._thunk.shape

    @property
    def ndim(self) -> int:
        return self._thunk.ndim

    @property
    def size(self) -> int:
        return self._thunk.size

    @property
    def dtype(self) -> np.dtype:
        return self._thunk.dtype

    @property
    def global_lo(self) -> int:
        """First global position (along axis 0) held by this process's tile."""
        return self._thunk.global_lo

    def torch(self) -> torch.Tensor:
        """This process's tile as a device tensor (no copy)."""
        return self._thunk.base

    def to_numpy(self, out: np.ndarray | None = None) -> np.ndarray:
        """Copies this process's tile to host memory (into ``out`` when given)."""
        t = self._thunk.base
        runtime.raise_pending()
        if out is None:
            return t.cpu().numpy() if t.dtype not in (torch.uint16, torch.uint32, torch.uint64) \
                else t.view(_SIGNED_VIEW[t.dtype]).cpu().numpy().view(self.dtype)
        dst = torch.from_numpy(out.view(_np_signed(out.dtype)))
        dst.copy_(t.view(dst.dtype) if t.dtype != dst.dtype else t, non_blocking=False)
        return out

    def __array__(self, dtype: Any = None, copy: Any = None) -> np.ndarray:
        a = self.to_numpy()
        return a.astype(dtype) if dtype is not None else a

    def sort(self, axis: Any = -1, kind: str = "quicksort", order: Any = None) -> None:
        """Sorts in place (``cupynumeric/_array/array.py:3774-3796``)."""
        self._thunk.sort(rhs=self._thunk, axis=axis, kind=kind, order=order)

    def argsort(self, axis: Any = -1, kind: str = "quicksort", order: Any = None) -> "ndarray":
        """Indices that sort the array (``cupynumeric/_array/array.py:3798-3825``)."""
        result = ndarray(self.shape, np.int64)
        result._thunk.sort(rhs=self._thunk, argsort=True, axis=axis, kind=kind, order=order)
        return result


_SIGNED_VIEW = {torch.uint16: torch.int16, torch.uint32: torch.int32, torch.uint64: torch.int64}


def _np_signed(dt: np.dtype) -> np.dtype:
    dt = np.dtype(dt)
    return {np.dtype(np.uint16): np.dtype(np.int16), np.dtype(np.uint32): np.dtype(np.int32),
            np.dtype(np.uint64): np.dtype(np.int64)}.get(dt, dt)


def array(obj: Any, global_lo: int = 0) -> ndarray:
    """Wraps a device tensor (no copy) or uploads a host array as this process's tile.

    ``global_lo`` is the tile's first position along axis 0 of the global array when several
    processes each hold one tile."""
    if isinstance(obj, ndarray):
        return obj
    if isinstance(obj, torch.Tensor):
        t = obj if obj.is_cuda else obj.to(runtime.device)
        return ndarray(tuple(t.shape), DeferredArray(t).dtype, DeferredArray(t, global_lo=global_lo))
    a = np.asarray(obj)
    tdt = to_torch_dtype(a.dtype)
    a = np.ascontiguousarray(a)
    host = torch.from_numpy(a.view(_np_signed(a.dtype)))
    dev = torch.empty(a.shape, dtype=host.dtype, device=runtime.device)
    dev.copy_(host, non_blocking=False)
    dev = dev.view(tdt) if dev.dtype != tdt else dev
    return ndarray(a.shape, a.dtype, DeferredArray(dev, global_lo=global_lo))
