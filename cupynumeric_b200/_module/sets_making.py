"""``unique``: the sorted distinct values of an array, with the signature and the restrictions of
``cupynumeric/_module/sets_making.py:27-103`` (optional outputs and ``axis`` are not supported
there either).  Sort, then keep the head of every run of equal keys; with several processes the
sort is the distributed one and each rank drops a leading value its lower neighbour already
holds, so the parts stay sorted, disjoint and in rank order."""
from __future__ import annotations

import ctypes
from typing import Any

import numpy as np
import torch
import torch.distributed as dist

from .. import _lib
from .._array import array, ndarray
from .._thunk.deferred import DeferredArray, to_numpy_dtype
from ..runtime import runtime
from .ssc_sorting import sort


def _unique_sorted_tile(t: torch.Tensor) -> torch.Tensor:
    lib = _lib.lib()
    n = t.numel()
    out = torch.empty_like(t)
    if n == 0:
        return out
    need = ctypes.c_size_t()
    _lib.check(lib.b2s_unique_workspace_bytes(n, ctypes.byref(need)), "b2s_unique_workspace_bytes")
    ws = runtime.workspace(need.value)
    count = ctypes.c_size_t()
    _lib.check(lib.b2s_unique_sorted(_lib.DTYPE_CODE[to_numpy_dtype(t.dtype)], t.data_ptr(), n, out.data_ptr(),
                                     ctypes.byref(count), ws.data_ptr(), ws.numel(), runtime.stream_handle()),
               "b2s_unique_sorted")
    return out[: count.value]


def _ties(x: torch.Tensor, y: torch.Tensor) -> bool:
    """Equality in the sort's sense: NaN ties with NaN, -0.0 with +0.0."""
    if x.dtype.is_floating_point:
        return bool(((x == y) | (torch.isnan(x) & torch.isnan(y))).item())
    return bool((x == y).item())


def unique(ar: Any, return_index: bool = False, return_inverse: bool = False, return_counts: bool = False,
           axis: int | None = None) -> ndarray:
    if return_index or return_inverse or return_counts or axis is not None:
        raise NotImplementedError("Keyword arguments for `unique` are not yet supported")
    a = array(ar)
    srt = sort(a, axis=None) if a.ndim != 1 else sort(a)
    part = _unique_sorted_tile(srt.torch().contiguous())
    if runtime.num_procs > 1:
        # (has data, last value) of every rank; drop my first value if the nearest lower rank
        # that holds data ends with a tie of it
        world, rank = dist.get_world_size(), dist.get_rank()
        has = torch.tensor([1 if part.numel() else 0], dtype=torch.int64, device=part.device)
        last = part[-1:].clone() if part.numel() else torch.zeros(1, dtype=part.dtype, device=part.device)
        all_has = [torch.zeros_like(has) for _ in range(world)]
        all_last = [torch.zeros_like(last) for _ in range(world)]
        dist.all_gather(all_has, has)
        dist.all_gather([t.view(torch.uint8) for t in all_last], last.view(torch.uint8))
        if part.numel():
            for r in range(rank - 1, -1, -1):
                if int(all_has[r].item()):
                    if _ties(part[:1], all_last[r]):
                        part = part[1:]
                    break
    return ndarray(tuple(part.shape), to_numpy_dtype(part.dtype), DeferredArray(part))
