"""Shared helpers of the GPU parity tests: call the C ABI on host arrays and compare bit for bit
with the CPU oracle."""
from __future__ import annotations

import ctypes

import numpy as np
import torch

from cupynumeric_b200 import _lib
from cupynumeric_b200._thunk.deferred import to_torch_dtype

_SIGNED = {np.dtype(np.uint16): np.int16, np.dtype(np.uint32): np.int32, np.dtype(np.uint64): np.int64}


def to_device(a: np.ndarray) -> torch.Tensor:
    a = np.ascontiguousarray(a)
    v = a.view(_SIGNED.get(a.dtype, a.dtype))
    return torch.from_numpy(v).cuda()


def to_host(t: torch.Tensor, dtype) -> np.ndarray:
    return t.cpu().numpy().view(dtype)


def cabi_local_sort(keys: np.ndarray, segment: int, argsort: bool, index_offset: int = 0,
                    ndim_is_1: bool = True, inplace: bool = False, want_keys_too: bool = False):
    """Calls ``b2s_local_sort`` straight through ctypes. Returns (keys_or_None, idx_or_None)."""
    lib = _lib.lib()
    keys = np.ascontiguousarray(keys).reshape(-1)
    code = _lib.DTYPE_CODE[keys.dtype]
    d_in = to_device(keys)
    n = keys.size
    d_out = d_in if inplace else torch.empty_like(d_in)
    d_idx = torch.empty(n, dtype=torch.int64, device="cuda") if argsort else None
    need = ctypes.c_size_t(0)
    _lib.check(lib.b2s_workspace_bytes(code, n, segment, int(argsort), ctypes.byref(need)), "ws")
    ws = torch.empty(max(need.value, 256), dtype=torch.uint8, device="cuda")
    write_keys = (not argsort) or want_keys_too
    st = lib.b2s_local_sort(code, d_in.data_ptr(), d_out.data_ptr() if write_keys else None,
                            d_idx.data_ptr() if argsort else None, n, segment, index_offset,
                            int(ndim_is_1), 1, ws.data_ptr(), ws.numel(),
                            torch.cuda.current_stream().cuda_stream)
    _lib.check(st, "b2s_local_sort")
    _lib.check(lib.b2s_check_status(ws.data_ptr(), torch.cuda.current_stream().cuda_stream), "status")
    return (to_host(d_out, keys.dtype) if write_keys else None,
            d_idx.cpu().numpy() if argsort else None)


def bits(a: np.ndarray) -> np.ndarray:
    """Bit pattern view for exact comparison of floats (NaN payloads, signed zeros)."""
    a = np.ascontiguousarray(a)
    if a.dtype.kind == "c":
        return a.view(np.uint32 if a.dtype.itemsize == 8 else np.uint64)
    return a.view({1: np.uint8, 2: np.uint16, 4: np.uint32, 8: np.uint64}[a.dtype.itemsize])


def assert_bit_equal(got: np.ndarray, want: np.ndarray, what: str = "") -> None:
    assert got.shape == want.shape, (what, got.shape, want.shape)
    gb, wb = bits(got), bits(want)
    if not np.array_equal(gb, wb):
        bad = np.flatnonzero(gb.reshape(-1) != wb.reshape(-1))
        raise AssertionError(f"{what}: {bad.size} of {gb.size} differ, first at {bad[:5]}: "
                             f"got {got.reshape(-1)[bad[:5]]} want {want.reshape(-1)[bad[:5]]}")


ALL_DTYPES = [np.bool_, np.int8, np.int16, np.int32, np.int64, np.uint8, np.uint16, np.uint32,
              np.uint64, np.float16, np.float32, np.float64]


def random_keys(rng: np.random.Generator, dtype, n: int, flavour: str = "full") -> np.ndarray:
    """Test inputs: ``full`` covers the whole value range (floats: random bit patterns with NaNs,
    infinities, denormals and signed zeros); ``small`` has few distinct values (many ties)."""
    dt = np.dtype(dtype)
    if dt == np.bool_:
        return rng.integers(0, 2, n).astype(np.bool_)
    if flavour == "small":
        vals = rng.integers(-100, 100, n)
        if dt.kind == "u":
            vals = np.abs(vals)
        if dt.kind == "f":
            out = (vals / 4).astype(dt)
            out[rng.integers(0, max(n, 1), n // 50)] = np.nan
            out[rng.integers(0, max(n, 1), n // 50)] = -0.0
            out[rng.integers(0, max(n, 1), n // 50)] = 0.0
            return out
        return vals.astype(dt)
    raw = rng.integers(0, 256, n * dt.itemsize, dtype=np.uint8).view(dt)
    return raw.copy()
