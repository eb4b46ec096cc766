"""The C-ABI library loads, exports every function the header declares, and its host-only
entry points behave (no kernel is launched here)."""
import ctypes
import re

import numpy as np
import pytest

from cupynumeric_b200 import _lib


def declared_functions():
    src = open(_lib.HEADER_PATH).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(b2s_[a-z0-9_]+)\s*\(", src)))


def test_header_declares_something():
    names = declared_functions()
    assert "b2s_local_sort" in names and "b2s_workspace_bytes" in names


def test_library_exports_every_declared_symbol():
    handle = ctypes.CDLL(_lib.LIB_PATH)
    for name in declared_functions():
        assert hasattr(handle, name), f"{name} declared in include/b200sort.h but not exported"


def test_binding_covers_every_declared_symbol():
    assert sorted(_lib.SIGNATURES) == declared_functions()
    _lib.lib()


def test_status_strings():
    lib = _lib.lib()
    seen = {lib.b2s_status_string(s) for s in range(7)}
    assert len(seen) == 7 and lib.b2s_status_string(0) == b"ok"
    assert lib.b2s_version() >= 100


@pytest.mark.parametrize("dtype", [np.int32, np.float32, np.uint64, np.float16, np.bool_])
def test_workspace_bytes_grows_with_problem(dtype):
    lib = _lib.lib()
    code = _lib.DTYPE_CODE[np.dtype(dtype)]
    out = ctypes.c_size_t(0)
    assert lib.b2s_workspace_bytes(code, 0, 0, 0, ctypes.byref(out)) == 0
    assert lib.b2s_workspace_bytes(code, 4096 * 10, 4096, 0, ctypes.byref(out)) == 0
    small = out.value
    assert lib.b2s_workspace_bytes(code, 1 << 24, 1 << 24, 0, ctypes.byref(out)) == 0
    keys_only = out.value
    assert lib.b2s_workspace_bytes(code, 1 << 24, 1 << 24, 1, ctypes.byref(out)) == 0
    pairs = out.value
    item = np.dtype(dtype).itemsize
    assert small < keys_only < pairs
    assert keys_only >= 2 * (1 << 24) * item and pairs >= 2 * (1 << 24) * (item + 4)


def test_workspace_bytes_rejects_bad_arguments():
    lib = _lib.lib()
    out = ctypes.c_size_t(0)
    assert lib.b2s_workspace_bytes(4, 10, 3, 0, ctypes.byref(out)) == 1      # volume % segment
    assert lib.b2s_workspace_bytes(4, 10, 0, 0, ctypes.byref(out)) == 1      # zero segment
    assert lib.b2s_workspace_bytes(99, 10, 10, 0, ctypes.byref(out)) == 6    # unknown dtype
    assert lib.b2s_workspace_bytes(4, 10, 10, 0, None) == 1


def test_local_sort_validates_before_touching_the_gpu():
    lib = _lib.lib()
    # empty tile: nothing to do, no pointers needed
    assert lib.b2s_local_sort(4, None, None, None, 0, 0, 0, 1, 0, None, 0, None) == 0
    assert lib.b2s_local_sort(4, None, None, None, 8, 8, 0, 1, 0, None, 0, None) == 1
    assert lib.b2s_local_sort(99, None, None, None, 8, 8, 0, 1, 0, None, 0, None) == 6
    fake = ctypes.c_void_p(4096)
    # missing / undersized workspace
    assert lib.b2s_local_sort(4, fake, fake, None, 8, 8, 0, 1, 0, None, 0, None) == 4
    assert lib.b2s_local_sort(4, fake, fake, None, 1 << 20, 1 << 20, 0, 1, 0, fake, 16, None) == 4
    # a 1-D call must be a single segment
    assert lib.b2s_local_sort(4, fake, fake, None, 8, 4, 0, 1, 0, fake, 1 << 20, None) == 1
