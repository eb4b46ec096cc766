"""Multi-GPU plumbing of the 1-D sort: one process per GPU, ``torch.distributed`` for the
rendezvous, NCCL (through ``b2s_dist_sort_1d``) for the data path.

Stands where Legate adds an NCCL communicator to the task and hands every point task its
``ncclComm_t`` (``cupynumeric/_thunk/_sort.py:89-90``, ``src/cupynumeric/sort/sort.cu:1923``)."""
from __future__ import annotations

import ctypes

import numpy as np
import torch
import torch.distributed as dist

from . import _lib
from ._thunk.deferred import to_numpy_dtype
from .runtime import runtime


class _Pool:
    """Allocator handed to the C ABI: device memory comes from torch's caching allocator and
    stays alive until the library returns it or the caller adopts it."""

    def __init__(self) -> None:
        self.live: dict[int, torch.Tensor] = {}
        self.alloc_cb = _lib.ALLOC_FN(self._alloc)
        self.free_cb = _lib.FREE_FN(self._free)

    def _alloc(self, _ctx, nbytes):
        try:
            t = torch.empty(max(int(nbytes), 256), dtype=torch.uint8, device=runtime.device)
        except Exception:
            return None
        self.live[t.data_ptr()] = t
        return t.data_ptr()

    def _free(self, _ctx, ptr):
        self.live.pop(ptr, None)

    def adopt(self, ptr: int) -> torch.Tensor:
        return self.live.pop(ptr)


_comm = None


def nccl_comm() -> int:
    """The process group's NCCL communicator for the sort library (created on first use: rank 0
    makes the unique id, ``torch.distributed`` broadcasts it)."""
    global _comm
    if _comm is None:
        lib = _lib.lib()
        ident = torch.zeros(128, dtype=torch.uint8)
        if dist.get_rank() == 0:
            buf = (ctypes.c_ubyte * 128)()
            _lib.check(lib.b2s_nccl_unique_id(buf), "b2s_nccl_unique_id")
            ident = torch.tensor(list(buf), dtype=torch.uint8)
        backend = dist.get_backend()
        ident = ident.to(runtime.device) if backend == "nccl" else ident
        dist.broadcast(ident, src=0)
        raw = bytes(ident.cpu().tolist())
        handle = ctypes.c_void_p()
        _lib.check(lib.b2s_nccl_comm_create(ctypes.byref(handle), dist.get_world_size(), raw, dist.get_rank()),
                   "b2s_nccl_comm_create")
        _comm = handle.value
    return _comm


def destroy_comm() -> None:
    global _comm
    if _comm is not None:
        _lib.lib().b2s_nccl_comm_destroy(_comm)
        _comm = None


def dist_sort_1d(tile: torch.Tensor, argsort: bool, global_lo: int):
    """Sorts the 1-D array whose rank-ordered tiles are ``tile`` on every process.  Returns this
    process's part of the result (values, or int64 global indices) and the global position of
    its first element."""
    lib = _lib.lib()
    assert tile.is_cuda and tile.ndim == 1 and tile.is_contiguous()
    np_dtype = to_numpy_dtype(tile.dtype)
    pool = _Pool()
    out_ptr, out_len, out_start = ctypes.c_void_p(), ctypes.c_size_t(), ctypes.c_int64()
    st = lib.b2s_dist_sort_1d(_lib.DTYPE_CODE[np_dtype], tile.data_ptr(), tile.numel(), int(global_lo), int(argsort),
                              nccl_comm(), dist.get_rank(), dist.get_world_size(),
                              ctypes.cast(pool.alloc_cb, ctypes.c_void_p), ctypes.cast(pool.free_cb, ctypes.c_void_p),
                              None, None, None, ctypes.byref(out_ptr), ctypes.byref(out_len),
                              ctypes.byref(out_start), runtime.stream_handle())
    _lib.check(st, "b2s_dist_sort_1d")
    raw = pool.adopt(out_ptr.value)
    res_dtype = torch.int64 if argsort else tile.dtype
    n = out_len.value
    result = raw[: n * res_dtype.itemsize].view(res_dtype)
    return result, int(out_start.value)


def rebalance_1d(part: torch.Tensor, part_start: int, out: torch.Tensor, out_start: int) -> None:
    """Moves the rank-ordered, variable-length parts of a distributed sort into fixed extents:
    afterwards ``out`` holds the elements ``[out_start, out_start + len(out))`` of the global
    sorted sequence."""
    lib = _lib.lib()
    assert out.is_contiguous() and part.dtype == out.dtype
    pool = _Pool()
    st = lib.b2s_dist_rebalance_1d(part.element_size(), part.data_ptr() if part.numel() else None, part.numel(),
                                   int(part_start), out.data_ptr() if out.numel() else None, out.numel(),
                                   int(out_start), nccl_comm(), dist.get_rank(), dist.get_world_size(),
                                   ctypes.cast(pool.alloc_cb, ctypes.c_void_p), ctypes.cast(pool.free_cb, ctypes.c_void_p),
                                   None, None, None, runtime.stream_handle())
    _lib.check(st, "b2s_dist_rebalance_1d")


def dist_sort_nd(tile: torch.Tensor, argsort: bool) -> torch.Tensor:
    """Sorts an N-D tile along its last axis when that axis is the one split over the processes
    (every process holds the same rows and a slice of each): all rows in one call, results in the
    tile's own extents."""
    lib = _lib.lib()
    assert tile.is_cuda and tile.is_contiguous() and tile.ndim >= 2
    np_dtype = to_numpy_dtype(tile.dtype)
    extent = tile.shape[-1]
    rows = tile.numel() // extent if extent else 0
    out = torch.empty(tile.shape, dtype=torch.int64 if argsort else tile.dtype, device=tile.device)
    pool = _Pool()
    st = lib.b2s_dist_sort_nd(_lib.DTYPE_CODE[np_dtype], tile.data_ptr() if tile.numel() else None,
                              out.data_ptr() if out.numel() else None, int(argsort), rows, extent, nccl_comm(), dist.get_rank(),
                              dist.get_world_size(), ctypes.cast(pool.alloc_cb, ctypes.c_void_p),
                              ctypes.cast(pool.free_cb, ctypes.c_void_p), None, None, None, runtime.stream_handle())
    _lib.check(st, "b2s_dist_sort_nd")
    return out
