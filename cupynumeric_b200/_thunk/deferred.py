"""Device-resident array thunk: the part of the reference's ``DeferredArray``
(``cupynumeric/_thunk/deferred.py:287``) that the SORT path touches.

``base`` is this process's dense, row-major tile of the global array (the whole array when one
process runs).  With several processes the global array is tiled along axis 0 in rank order,
which is how Legate tiles the stores of this task for the shapes in scope: 1-D arrays into
contiguous ranges, N-D arrays into row blocks.
"""
from __future__ import annotations

from typing import Any

import numpy as np
import torch

from ..runtime import runtime

_NP2TORCH = {
    np.dtype(np.bool_): torch.bool, np.dtype(np.int8): torch.int8, np.dtype(np.int16): torch.int16,
    np.dtype(np.int32): torch.int32, np.dtype(np.int64): torch.int64, np.dtype(np.uint8): torch.uint8,
    np.dtype(np.uint16): torch.uint16, np.dtype(np.uint32): torch.uint32,
    np.dtype(np.uint64): torch.uint64, np.dtype(np.float16): torch.float16,
    np.dtype(np.float32): torch.float32, np.dtype(np.float64): torch.float64,
    np.dtype(np.complex64): torch.complex64, np.dtype(np.complex128): torch.complex128,
}
_TORCH2NP = {v: k for k, v in _NP2TORCH.items()}


def to_torch_dtype(dt: Any) -> torch.dtype:
    try:
        return _NP2TORCH[np.dtype(dt)]
    except (KeyError, TypeError):
        # same failure mode as the reference's store conversion (cupynumeric/runtime.py:345-348)
        raise TypeError(f"cuPyNumeric does not support dtype={dt}")


def to_numpy_dtype(dt: torch.dtype) -> np.dtype:
    return _TORCH2NP[dt]


class DeferredArray:
    def __init__(self, base: torch.Tensor | None, dtype: np.dtype | None = None,
                 shape: tuple[int, ...] | None = None, global_lo: int = 0, tiled_axis: int = 0) -> None:
        self.base = base
        self._dtype = np.dtype(dtype) if dtype is not None else to_numpy_dtype(base.dtype)
        self._shape = tuple(shape) if shape is not None else tuple(base.shape)
        # position of this tile along axis 0 of the global array (1-D: first global index held)
        self.global_lo = int(global_lo)
        # axis along which the processes' tiles are laid out (0 unless a view swapped it away)
        self.tiled_axis = int(tiled_axis)

    # ---- geometry ----
    @property
    def shape(self) -> tuple[int, ...]:
        return tuple(self.base.shape) if self.base is not None else self._shape

    @property
    def ndim(self) -> int:
        return len(self.shape)

    @property
    def size(self) -> int:
        return int(np.prod(self.shape, dtype=np.int64)) if self.ndim else 1

    @property
    def dtype(self) -> np.dtype:
        return self._dtype

    # ---- the views the sort dispatch needs ----
    def reshape(self, newshape: tuple[int, ...], order: str = "C") -> "DeferredArray":
        """C-order reshape.  Flattening a row-tiled array keeps the tiles contiguous in the flat
        index space, so the tile offset scales by the number of elements per row."""
        lo = self.global_lo
        if self.ndim > 1 and len(newshape) == 1 and self.tiled_axis == 0 and self.shape[0] > 0:
            lo = self.global_lo * (self.size // self.shape[0])
        return DeferredArray(self.base.contiguous().reshape(newshape), global_lo=lo)

    def swapaxes(self, axis1: int, axis2: int) -> "DeferredArray":
        a1, a2 = axis1 % max(self.ndim, 1), axis2 % max(self.ndim, 1)
        tiled = a2 if self.tiled_axis == a1 else a1 if self.tiled_axis == a2 else self.tiled_axis
        return DeferredArray(self.base.swapaxes(axis1, axis2), global_lo=self.global_lo, tiled_axis=tiled)

    def copy(self, rhs: "DeferredArray", deep: bool = True) -> None:
        """Fills this thunk with a dense row-major copy of ``rhs``."""
        self.base = rhs.base.contiguous() if not deep else rhs.base.clone(memory_format=torch.contiguous_format)
        self.global_lo, self.tiled_axis = rhs.global_lo, rhs.tiled_axis

    # ---- SORT ----
    def sort(self, rhs: "DeferredArray", argsort: bool = False, axis: int | None = -1,
             kind: str = "quicksort", order: Any = None) -> None:
        """Same checks, in the same order, as ``DeferredArray.sort``
        (``cupynumeric/_thunk/deferred.py:5453-5474``): only ``kind == "stable"`` requests a
        stable sort; ``order`` is not supported; an out-of-range axis is a ``ValueError``."""
        from ._sort import sort_deferred

        stable = kind == "stable"
        if order is not None:
            raise NotImplementedError(
                "cuPyNumeric does not support sorting with 'order' as ndarray only supports numeric values")
        if axis is not None and (axis >= rhs.ndim or axis < -rhs.ndim):
            raise ValueError("invalid axis")
        sort_deferred(self, rhs, argsort, axis, stable)


    def searchsorted(self, rhs: "DeferredArray", v: "DeferredArray", side: str = "left") -> None:
        """Fills this int64 thunk (shaped like ``v``) with insertion positions of ``v`` in the
        sorted 1-D array ``rhs`` whose tiles may span the processes.  Follows
        ``DeferredArray.searchsorted`` (``cupynumeric/_thunk/deferred.py:5425-5451``): pre-fill
        with ``rhs`` global size (left) or 0 (right), per-tile contributions, MIN / MAX over
        ranks.  ``v`` is the same on every process (broadcast constraint of the reference)."""
        import torch.distributed as dist

        from .. import _lib

        lib = _lib.lib()
        is_left = side == "left"
        tile = rhs.base.contiguous()
        vals = v.base.contiguous()
        assert vals.dtype == tile.dtype, "searchsorted: the caller brings both arrays to one dtype"
        global_size = tile.numel()
        if runtime.num_procs > 1:
            t = torch.tensor([global_size], dtype=torch.int64, device=tile.device)
            dist.all_reduce(t)
            global_size = int(t.item())
        out = torch.full(vals.shape, global_size if is_left else 0, dtype=torch.int64, device=tile.device)
        _lib.check(lib.b2s_searchsorted(_lib.DTYPE_CODE[to_numpy_dtype(tile.dtype)],
                                        tile.data_ptr() if tile.numel() else None, tile.numel(), rhs.global_lo,
                                        vals.data_ptr() if vals.numel() else None, vals.numel(), int(is_left),
                                        out.data_ptr() if out.numel() else None, runtime.stream_handle()),
                   "b2s_searchsorted")
        if runtime.num_procs > 1:
            dist.all_reduce(out, op=dist.ReduceOp.MIN if is_left else dist.ReduceOp.MAX)
        self.base = out


def create_deferred_thunk(shape: tuple[int, ...], dtype: Any) -> DeferredArray:
    """An output thunk whose device memory is attached by the task that fills it."""
    return DeferredArray(None, dtype=np.dtype(dtype), shape=tuple(shape))
