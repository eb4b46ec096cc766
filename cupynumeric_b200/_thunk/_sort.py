"""Host-side dispatch of the SORT task: axis handling and task construction.

Mirrors the routing of ``cupynumeric/_thunk/_sort.py:37-136`` (same function names and
argument meaning) on top of device-resident tiles instead of Legate stores:

* ``sort_deferred``  0-D / ``axis=None`` / last-axis / other-axis routing   (ref ``:110-136``)
* ``sort_flattened`` ``axis=None`` on an N-D array: sort the C-order flattening (ref ``:37-47``)
* ``sort_swapped``   other axes: swap to last, dense copy, sort, swap back   (ref ``:50-76``)
* ``sort_task``      one point task per process on its tile                  (ref ``:79-107``)
"""
from __future__ import annotations

import ctypes

import numpy as np
import torch
from numpy.exceptions import AxisError
from numpy.lib.array_utils import normalize_axis_index

from .. import _lib
from ..runtime import runtime
from .deferred import DeferredArray, create_deferred_thunk, to_numpy_dtype


def local_sort_tile(tile: torch.Tensor, argsort: bool, stable: bool, index_offset: int = 0,
                    out: torch.Tensor | None = None) -> torch.Tensor:
    """Runs the point task body on one dense row-major tile: sorts along the last axis.

    This is the call the reference's ``SortImplBody<GPU>`` makes into ``local_sort``
    (``src/cupynumeric/sort/sort.cu:1881-1891``), here into ``b2s_local_sort``.
    """
    lib = _lib.lib()
    assert tile.is_cuda and tile.is_contiguous()
    code = _lib.DTYPE_CODE[to_numpy_dtype(tile.dtype)]
    volume = tile.numel()
    segment = tile.shape[-1] if tile.ndim else 1
    if out is None:
        out = torch.empty(tile.shape, dtype=torch.int64 if argsort else tile.dtype, device=tile.device)
    if volume == 0:
        return out
    need = ctypes.c_size_t(0)
    _lib.check(lib.b2s_workspace_bytes(code, volume, segment, int(argsort), ctypes.byref(need)),
               "b2s_workspace_bytes")
    ws = runtime.workspace(need.value)
    st = lib.b2s_local_sort(code, tile.data_ptr(), None if argsort else out.data_ptr(),
                            out.data_ptr() if argsort else None, volume, segment, int(index_offset),
                            int(tile.ndim == 1), int(stable), ws.data_ptr(), ws.numel(),
                            runtime.stream_handle())
    _lib.check(st, "b2s_local_sort")
    if tile.dtype != torch.complex128:  # (its inner sorts keep their control blocks elsewhere)
        runtime.note_sort(ws)
    return out


def sort_flattened(output: DeferredArray, input: DeferredArray, argsort: bool, stable: bool) -> None:
    flat = input.reshape((input.size,), order="C")
    result = create_deferred_thunk(flat.shape, dtype=output.dtype)
    sort_deferred(result, flat, argsort, stable=stable)
    output.base, output.global_lo, output.tiled_axis = result.base, result.global_lo, result.tiled_axis


def sort_swapped(output: DeferredArray, input: DeferredArray, argsort: bool, sort_axis: int,
                 stable: bool) -> None:
    sort_axis = normalize_axis_index(sort_axis, input.ndim)
    last = input.ndim - 1
    moved = create_deferred_thunk(input.swapaxes(sort_axis, last).shape, dtype=input.dtype)
    moved.copy(input.swapaxes(sort_axis, last), deep=True)
    if argsort:
        result = create_deferred_thunk(moved.shape, dtype=output.dtype)
        sort_deferred(result, moved, argsort, stable=stable)
        back = result.swapaxes(last, sort_axis)
    else:
        sort_deferred(moved, moved, argsort, stable=stable)
        back = moved.swapaxes(last, sort_axis)
    output.base, output.global_lo, output.tiled_axis = back.base, back.global_lo, back.tiled_axis


def sort_task(output: DeferredArray, input: DeferredArray, argsort: bool, stable: bool) -> None:
    """One point task per process on its tile; the tile's last axis is the sort axis.

    A 1-D array held by several processes gets an "unbound" output: each process ends up with
    however many elements fall between its splitters (ref ``:87,99-103``); N-D arrays are tiled
    by rows, so every segment is local and no exchange happens (the reference reaches the same
    state: ``need_distributed_sort == false``, ``src/cupynumeric/sort/sort.cu:1825``).
    """
    tile = input.base if input.base.is_contiguous() else input.base.contiguous()
    if runtime.num_procs > 1 and input.ndim > 1 and input.tiled_axis == input.ndim - 1:
        sort_split_axis(output, input, tile, argsort)
        return
    uses_unbound_output = runtime.num_procs > 1 and input.ndim == 1
    if uses_unbound_output:
        from .._dist import dist_sort_1d

        output.base, output.global_lo = dist_sort_1d(tile, argsort, input.global_lo)
        return
    # write straight into the output's memory when it is already there (in-place ndarray.sort)
    out = output.base if (not argsort and output.base is not None and output.base.is_contiguous()
                          and output.base.shape == tile.shape and output.base.dtype == tile.dtype) else None
    output.base = local_sort_tile(tile, argsort, stable,
                                  index_offset=input.global_lo if input.ndim == 1 else 0, out=out)
    output.global_lo, output.tiled_axis = input.global_lo, input.tiled_axis


def sort_split_axis(output: DeferredArray, input: DeferredArray, tile: torch.Tensor, argsort: bool) -> None:
    """N-D tile whose sort (last) axis is the one split over the processes: every row is a 1-D
    array spanning the ranks, and the output store is bound and aligned with the input, so every
    rank must end up with exactly its own extent of every sorted row (the reference:
    sample_sort_nccl_nd over all segments + rebalance_data,
    ``src/cupynumeric/sort/sort.cu:1759-1773,799-1261``).  With at least as many rows as ranks all
    rows go through one call (``b2s_dist_sort_nd``: rows dealt out, completed by one exchange,
    sorted, returned by another).  Fewer rows than ranks would leave ranks idle that way: each row
    then takes the distributed 1-D sort and is moved back into this rank's extent."""
    from .._dist import dist_sort_1d, dist_sort_nd, rebalance_1d

    extent = tile.shape[-1]
    rows = tile.reshape(-1, extent)
    if rows.shape[0] >= runtime.num_procs:
        out = dist_sort_nd(rows, argsort)
    else:
        out = torch.empty(rows.shape, dtype=torch.int64 if argsort else tile.dtype, device=tile.device)
        for i in range(rows.shape[0]):
            part, start = dist_sort_1d(rows[i], argsort, input.global_lo)
            rebalance_1d(part, start, out[i], input.global_lo)
    output.base = out.reshape(tile.shape)
    output.global_lo, output.tiled_axis = input.global_lo, input.tiled_axis


def sort_deferred(output: DeferredArray, input: DeferredArray, argsort: bool, axis: int | None = -1,
                  stable: bool = False) -> None:
    if input.ndim == 0:
        if axis is not None:
            raise AxisError(axis, input.ndim)
        output.base = input.base
        return
    if axis is None and input.ndim > 1:
        sort_flattened(output, input, argsort, stable)
        return
    computed_axis = 0 if axis is None else normalize_axis_index(axis, input.ndim)
    if computed_axis == input.ndim - 1:
        sort_task(output, input, argsort, stable)
    else:
        sort_swapped(output, input, argsort, computed_axis, stable)
