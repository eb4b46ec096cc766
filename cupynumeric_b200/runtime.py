"""Process-level state of the host layer: which GPU this process drives, how many processes
take part (one per GPU), and the scratch memory handed to the kernels.

Plays the role the Legate runtime plays for the reference's SORT task: it owns device memory
(through torch's caching allocator, the stand-in for Legate's framebuffer pool,
``src/cupynumeric/mapper.cc:635-643``), the stream, and the communicator
(``cupynumeric/_thunk/_sort.py:87-92``).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from . import _lib


class Runtime:
    def __init__(self) -> None:
        self._ws: dict[int, torch.Tensor] = {}
        self._sticky: dict[int, torch.Tensor] = {}
        self._comm = None

    # --- topology -------------------------------------------------------------------------
    @property
    def num_procs(self) -> int:
        return dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1

    @property
    def rank(self) -> int:
        return dist.get_rank() if dist.is_available() and dist.is_initialized() else 0

    @property
    def num_gpus(self) -> int:
        return self.num_procs if torch.cuda.is_available() else 0

    @property
    def device(self) -> torch.device:
        if not torch.cuda.is_available():
            raise RuntimeError("cupynumeric_b200 needs a CUDA device: the sort kernels have no CPU path")
        return torch.device("cuda", torch.cuda.current_device())

    def stream_handle(self) -> int:
        return torch.cuda.current_stream().cuda_stream

    # --- scratch memory -------------------------------------------------------------------
    def workspace(self, nbytes: int) -> torch.Tensor:
        """A 256-byte aligned device buffer of at least ``nbytes``, reused between calls on the
        same device (calls on one stream are ordered, so reuse is safe)."""
        dev = torch.cuda.current_device()
        cur = self._ws.get(dev)
        if cur is None or cur.numel() < nbytes:
            self._ws.pop(dev, None)
            cur = None
            cur = torch.empty(max(int(nbytes), 1 << 16), dtype=torch.uint8, device=self.device)
            assert cur.data_ptr() % 256 == 0
            self._ws[dev] = cur
        return cur

    def release_workspace(self) -> None:
        self._ws.clear()

    # --- device-side status of the sorts enqueued so far ------------------------------------
    def note_sort(self, ws: torch.Tensor) -> None:
        """Folds the status word at the head of a workspace (0, or the code a kernel left when a
        bounded wait ran out) into a per-device word that survives the workspace's reuse.  Stream
        ordered, no synchronisation."""
        dev = torch.cuda.current_device()
        acc = self._sticky.get(dev)
        if acc is None:
            acc = self._sticky[dev] = torch.zeros(1, dtype=torch.int32, device=self.device)
        torch.maximum(acc, ws[:4].view(torch.int32), out=acc)

    def raise_pending(self) -> None:
        """Called where a result reaches the host: raises if any sort since the last call reported
        a device-side failure (role of CUPYNUMERIC_CHECK_CUDA_STREAM in the reference's task
        bodies, ``src/cupynumeric/cuda_help.h:291-302``)."""
        acc = self._sticky.get(torch.cuda.current_device()) if torch.cuda.is_available() else None
        if acc is None:
            return
        status = int(acc.item())
        if status != 0:
            acc.zero_()
            raise _lib.B2SError(status, "a sort kernel")


runtime = Runtime()
