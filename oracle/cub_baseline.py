"""MEASUREMENT INFRASTRUCTURE: ctypes front-end of ``cub_baseline.cu`` - the CCCL library sorts
the reference's GPU variant calls (``src/cupynumeric/sort/cub_sort.cuh:57-184``), timed by the
benchmark beside the hand-written kernels on the same GPU.  Not part of the product."""
from __future__ import annotations

import ctypes
import os
import subprocess

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libcub_baseline.so")
_lib = None

SUPPORTED = {"int32": 4, "int64": 5, "uint32": 8, "uint64": 9, "float32": 11, "float64": 12}


def build(force: bool = False) -> str:
    src = os.path.join(_HERE, "cub_baseline.cu")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "-s", "cub"], check=True)
    return _SO


def _load():
    global _lib
    if _lib is None:
        import torch  # noqa: F401  (loads the CUDA runtime the library links against)
        lib = ctypes.CDLL(_SO)
        lib.cubb_temp_bytes.restype = ctypes.c_int
        lib.cubb_temp_bytes.argtypes = [ctypes.c_int, ctypes.c_size_t, ctypes.c_size_t, ctypes.c_int,
                                        ctypes.POINTER(ctypes.c_size_t)]
        lib.cubb_sort.restype = ctypes.c_int
        lib.cubb_sort.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                  ctypes.c_size_t, ctypes.c_size_t, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p]
        _lib = lib
    return _lib


def available() -> bool:
    return os.path.exists(_SO)


def time_sort(tile, argsort: bool, steps: int = 5, warmup: int = 2, between=None):
    """Times the library sort on a device tensor (last axis = sort axis).  Returns (ms per step,
    result tensor).  ``tile`` is a torch CUDA tensor of a supported dtype.  ``between`` (a callable,
    e.g. an L2 flush for inputs that fit the cache) runs before every timed step, outside the timed
    interval; without it the steps are timed back to back."""
    import torch

    lib = _load()
    name = str(tile.dtype).replace("torch.", "")
    code = SUPPORTED[name]
    volume, segment = tile.numel(), tile.shape[-1]
    need = ctypes.c_size_t()
    rc = lib.cubb_temp_bytes(code, volume, segment, int(argsort), ctypes.byref(need))
    if rc != 0:
        raise RuntimeError(f"cubb_temp_bytes failed with CUDA error {rc}")
    temp = torch.empty(max(need.value, 256), dtype=torch.uint8, device=tile.device)
    keys_out = torch.empty_like(tile)
    idx_in = torch.empty(volume, dtype=torch.int64, device=tile.device) if argsort else None
    idx_out = torch.empty(tile.shape, dtype=torch.int64, device=tile.device) if argsort else None
    stream = torch.cuda.current_stream().cuda_stream

    def call():
        rc = lib.cubb_sort(code, tile.data_ptr(), keys_out.data_ptr(), idx_in.data_ptr() if argsort else None,
                           idx_out.data_ptr() if argsort else None, volume, segment, temp.data_ptr(), temp.numel(), stream)
        if rc != 0:
            raise RuntimeError(f"cubb_sort failed with CUDA error {rc}")

    for _ in range(warmup):
        call()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if between is not None:
        ms = 0.0
        for _ in range(steps):
            between()
            e0.record()
            call()
            e1.record()
            torch.cuda.synchronize()
            ms += e0.elapsed_time(e1)
        return ms / steps, (idx_out if argsort else keys_out)
    e0.record()
    for _ in range(steps):
        call()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps, (idx_out if argsort else keys_out)
