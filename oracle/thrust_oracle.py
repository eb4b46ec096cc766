"""TEST INFRASTRUCTURE: ctypes front-end of ``oracle_thrust.cpp`` (the reference's CPU/OMP
SORT arithmetic, ``src/cupynumeric/sort/sort_cpu.inl:52-85``, through Thrust's host and
OpenMP back-ends)."""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "liboracle_thrust.so")
_lib = None

# numbering shared with include/b200sort.h (b2s_dtype_t)
DTYPE_CODE = {
    np.dtype(np.bool_): 1, np.dtype(np.int8): 2, np.dtype(np.int16): 3, np.dtype(np.int32): 4,
    np.dtype(np.int64): 5, np.dtype(np.uint8): 6, np.dtype(np.uint16): 7, np.dtype(np.uint32): 8,
    np.dtype(np.uint64): 9, np.dtype(np.float16): 10, np.dtype(np.float32): 11,
    np.dtype(np.float64): 12, np.dtype(np.complex64): 13, np.dtype(np.complex128): 14,
}


def build(force: bool = False) -> str:
    """Compile the oracle with g++ (``oracle/Makefile``); returns the path of the library."""
    src = os.path.join(_HERE, "oracle_thrust.cpp")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "-s"], check=True)
    return _SO


def _load():
    global _lib
    if _lib is None:
        if not os.path.exists(_SO):
            build()
        _lib = ctypes.CDLL(_SO)
        _lib.oracle_sort.restype = ctypes.c_int
        _lib.oracle_sort.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t,
                                     ctypes.c_size_t, ctypes.c_int64, ctypes.c_int, ctypes.c_int,
                                     ctypes.c_int, ctypes.c_int]
    return _lib


def set_num_threads(n: int) -> None:
    """Sets the thread count of the OpenMP back-end for later calls."""
    lib = _load()
    lib.oracle_set_num_threads.argtypes = [ctypes.c_int]
    lib.oracle_set_num_threads.restype = None
    lib.oracle_set_num_threads(int(n))


def num_threads() -> int:
    """Threads the OpenMP back-end will use (OMP_NUM_THREADS or all cores)."""
    return int(_load().oracle_num_threads())


def thrust_task_sort(keys: np.ndarray, segment: int, argsort: bool, index_offset: int = 0,
                     ndim_is_1: bool = True, stable: bool = True, backend: str = "host",
                     nan_mode: str | None = None):
    """Run the reference's CPU (``backend="host"``) or OpenMP (``"omp"``) arithmetic on one tile.

    Returns ``(sorted_keys, indices_or_None)``.  ``nan_mode``: ``"literal"`` keeps the
    reference's raw ``<``; ``"nan_last"`` uses the NaN-last comparator; ``None`` picks
    ``"nan_last"`` only when the input holds a NaN (both agree otherwise).
    """
    lib = _load()
    keys = np.ascontiguousarray(keys).reshape(-1)
    work = keys.copy()  # the reference copies the input first (sort_cpu.inl:1020-1026)
    idx = np.empty(keys.size, dtype=np.int64) if argsort else None
    if nan_mode is None:
        has_nan = keys.dtype.kind == "f" and bool(np.isnan(keys).any())
        nan_mode = "nan_last" if has_nan else "literal"
    rc = lib.oracle_sort(DTYPE_CODE[keys.dtype], work.ctypes.data,
                         idx.ctypes.data if argsort else None, keys.size, int(segment),
                         int(index_offset), int(ndim_is_1), int(stable),
                         1 if backend == "omp" else 0, 1 if nan_mode == "nan_last" else 0)
    if rc != 0:
        raise ValueError(f"oracle_sort: unsupported dtype {keys.dtype}")
    return work, idx
