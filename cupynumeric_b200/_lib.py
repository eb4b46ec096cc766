"""ctypes binding of ``libb200sort.so`` (the C ABI declared in ``include/b200sort.h``).

There is no fallback: if the CUDA library is missing or a symbol is absent the import of the
binding raises, and every call that returns a non-zero status raises ``B2SError``.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(_HERE, "csrc")
# B2S_LIB_PATH selects another build of the same library (e.g. a tuning variant)
LIB_PATH = os.environ.get("B2S_LIB_PATH") or os.path.join(CSRC, "libb200sort.so")
HEADER_PATH = os.path.join(os.path.dirname(_HERE), "include", "b200sort.h")

# b2s_dtype_t
DTYPE_CODE = {
    np.dtype(np.bool_): 1, np.dtype(np.int8): 2, np.dtype(np.int16): 3, np.dtype(np.int32): 4,
    np.dtype(np.int64): 5, np.dtype(np.uint8): 6, np.dtype(np.uint16): 7, np.dtype(np.uint32): 8,
    np.dtype(np.uint64): 9, np.dtype(np.float16): 10, np.dtype(np.float32): 11,
    np.dtype(np.float64): 12, np.dtype(np.complex64): 13, np.dtype(np.complex128): 14,
}

B2S_OK = 0
# b2s_kernel_kind_t
K_HIST, K_SCAN, K_SWEEP, K_FIXUP, K_SEGSORT, K_UNIT, K_DIST, K_MERGE, K_XCHG = range(9)
STATUS_NAMES = {0: "B2S_OK", 1: "B2S_ERR_INVALID_ARG", 2: "B2S_ERR_CUDA", 3: "B2S_ERR_NCCL",
                4: "B2S_ERR_WORKSPACE", 5: "B2S_ERR_TIMEOUT", 6: "B2S_ERR_UNSUPPORTED"}


class B2SError(RuntimeError):
    def __init__(self, status: int, where: str):
        self.status = status
        msg = STATUS_NAMES.get(status, str(status))
        try:
            msg += ": " + lib().b2s_status_string(status).decode()
        except Exception:  # pragma: no cover
            pass
        super().__init__(f"{where} failed with {msg}")


def build_native(jobs: int = 8, force: bool = False) -> str:
    """Compiles the CUDA library in-tree for sm_100a (``csrc/Makefile``)."""
    env = dict(os.environ)
    nccl_inc, nccl_lib = nccl_paths()
    if nccl_inc:
        env["NCCL_INC"] = nccl_inc
        env["NCCL_LIB"] = nccl_lib
    if force:
        subprocess.run(["make", "-C", CSRC, "clean"], check=True, env=env, stdout=subprocess.DEVNULL)
    subprocess.run(["make", "-C", CSRC, f"-j{jobs}", "-s"], check=True, env=env)
    return LIB_PATH


def nccl_paths():
    """Include and library directories of the NCCL that torch itself loads."""
    try:
        import nvidia.nccl as _n  # type: ignore
        root = list(_n.__path__)[0]
        inc, libdir = os.path.join(root, "include"), os.path.join(root, "lib")
        if os.path.exists(os.path.join(inc, "nccl.h")):
            return inc, libdir
    except Exception:
        pass
    if os.path.exists("/usr/include/nccl.h"):
        return "/usr/include", "/usr/lib/x86_64-linux-gnu"
    return None, None


# callback types of b2s_dist_sort_1d
ALLOC_FN = ctypes.CFUNCTYPE(ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t)
FREE_FN = ctypes.CFUNCTYPE(None, ctypes.c_void_p, ctypes.c_void_p)
BARRIER_FN = ctypes.CFUNCTYPE(None, ctypes.c_void_p)

# layout of one sample record (see include/b200sort.h)
SAMPLE_DTYPE = np.dtype([("okey", np.uint64), ("okey_lo", np.uint64), ("pos", np.int64), ("weight", np.int64),
                         ("rank", np.int32), ("pad", np.int32)])


class CommOps(ctypes.Structure):
    """b2s_comm_ops: the collectives table of the distributed calls."""
    _fields_ = [("ctx", ctypes.c_void_p), ("all_gather", ctypes.c_void_p), ("barrier", ctypes.c_void_p),
                ("exchange", ctypes.c_void_p)]

_lib = None

_P, _SZ, _I, _I64 = ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int, ctypes.c_int64

# name -> (restype, argtypes); must list every function include/b200sort.h declares
SIGNATURES = {
    "b2s_status_string": (ctypes.c_char_p, [_I]),
    "b2s_version": (_I, []),
    "b2s_workspace_bytes": (_I, [_I, _SZ, _SZ, _I, ctypes.POINTER(_SZ)]),
    "b2s_local_sort": (_I, [_I, _P, _P, _P, _SZ, _SZ, _I64, _I, _I, _P, _SZ, _P]),
    "b2s_check_status": (_I, [_P, _P]),
    "b2s_selftest_wait_timeout": (_I, [_P, _SZ, _P]),
    "b2s_local_sort_noalloc": (_I, [_I, _P, _P, _P, _SZ, _SZ, _I64, _I, _P]),
    "b2s_noalloc_check_status": (_I, [_P]),
    "b2s_dist_sort_1d": (_I, [_I, _P, _SZ, _I64, _I, _P, _I, _I, _P, _P, _P, _P, _P,
                               ctypes.POINTER(_P), ctypes.POINTER(_SZ), ctypes.POINTER(_I64), _P]),
    "b2s_dist_sort_1d_ops": (_I, [_I, _P, _SZ, _I64, _I, _P, _I, _I, _P, _P, _P, _P, _P,
                                   ctypes.POINTER(_P), ctypes.POINTER(_SZ), ctypes.POINTER(_I64), _P]),
    "b2s_dist_rebalance_1d": (_I, [_SZ, _P, _SZ, _I64, _P, _SZ, _I64, _P, _I, _I, _P, _P, _P, _P, _P, _P]),
    "b2s_dist_rebalance_1d_ops": (_I, [_SZ, _P, _SZ, _I64, _P, _SZ, _I64, _P, _I, _I, _P, _P, _P, _P, _P, _P]),
    "b2s_dist_sort_nd_ops": (_I, [_I, _P, _P, _I, _SZ, _SZ, _P, _I, _I, _P, _P, _P, _P, _P, _P]),
    "b2s_dist_sort_nd": (_I, [_I, _P, _P, _I, _SZ, _SZ, _P, _I, _I, _P, _P, _P, _P, _P, _P]),
    "b2s_partition_workspace_bytes": (_I, [ctypes.POINTER(_SZ)]),
    "b2s_partition_1d": (_I, [_I, _P, _P, _P, _SZ, _SZ, _I64, _P, _SZ, _P]),
    "b2s_lexsort_workspace_bytes": (_I, [_I, _P, _SZ, _SZ, ctypes.POINTER(_SZ)]),
    "b2s_lexsort": (_I, [_I, _P, _P, _P, _SZ, _SZ, _P, _SZ, _P]),
    "b2s_nccl_comm_ops": (_I, [_P, _P, _I, _I, _P]),
    "b2s_nccl_comm_ops_release": (None, [_P]),
    "b2s_thread_comm_create": (_I, [_I, _P]),
    "b2s_thread_comm_destroy": (None, [_P]),
    "b2s_kway_merge_workspace_bytes": (_I, [_SZ, _I, ctypes.POINTER(_SZ)]),
    "b2s_kway_merge": (_I, [_I, _I, _P, _P, _P, _P, _P, _SZ, _P]),
    "b2s_nccl_unique_id": (_I, [_P]),
    "b2s_nccl_comm_create": (_I, [ctypes.POINTER(_P), _I, _P, _I]),
    "b2s_nccl_comm_destroy": (_I, [_P]),
    "b2s_samples_per_rank": (_I, []),
    "b2s_host_sample_position": (ctypes.c_longlong, [ctypes.c_longlong, ctypes.c_longlong, ctypes.c_longlong]),
    "b2s_host_sample_weight": (ctypes.c_longlong, [ctypes.c_longlong, ctypes.c_longlong, ctypes.c_longlong]),
    "b2s_host_sort_samples": (None, [_P, _SZ]),
    "b2s_host_select_splitters": (_I, [_P, _SZ, _I, _P]),
    "b2s_host_bucket_of": (_I, [_P, _I, _I, ctypes.c_ulonglong, ctypes.c_ulonglong, ctypes.c_longlong]),
    "b2s_searchsorted": (_I, [_I, _P, _SZ, _I64, _P, _SZ, _I, _P, _P]),
    "b2s_unique_workspace_bytes": (_I, [_SZ, ctypes.POINTER(_SZ)]),
    "b2s_unique_sorted": (_I, [_I, _P, _SZ, _P, ctypes.POINTER(_SZ), _P, _SZ, _P]),
    "b2s_profile_enable": (_I, [_I]),
    "b2s_profile_read": (_I, [_I, ctypes.POINTER(ctypes.c_double), ctypes.POINTER(ctypes.c_ulonglong)]),
    "b2s_profile_durations": (_I, [_I, ctypes.POINTER(ctypes.c_float), ctypes.c_size_t, ctypes.POINTER(ctypes.c_size_t)]),
    "b2s_launch_count": (ctypes.c_ulonglong, [_I]),
}


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -c 'import __graft_entry__ as g; g.build()'` "
                "(there is no CPU or library fallback for the sort kernels)")
        # torch loads the CUDA runtime and NCCL this library links against
        import torch  # noqa: F401
        handle = ctypes.CDLL(LIB_PATH, mode=ctypes.RTLD_GLOBAL)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)  # AttributeError if the symbol is not exported
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def check(status: int, where: str) -> None:
    if status != B2S_OK:
        raise B2SError(status, where)
