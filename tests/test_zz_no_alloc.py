"""The allocation-free entry point: ``b2s_local_sort_noalloc`` keeps its scratch in a fixed device
array inside the library, for callers that cannot allocate device memory themselves (a task body
under a runtime that forbids cudaMalloc while tasks run, a thread whose pool is exhausted).  Its
output must equal the regular entry point's, bit for bit, also when the shared scratch still
holds the previous call's contents."""
import ctypes

import numpy as np
import pytest
import torch

from cupynumeric_b200 import _lib
from tests.helpers import assert_bit_equal, cabi_local_sort, random_keys, to_device, to_host

pytestmark = pytest.mark.gpu


def noalloc_sort(keys: np.ndarray, segment: int, argsort: bool, index_offset: int = 0, ndim_is_1: bool = True):
    lib = _lib.lib()
    keys = np.ascontiguousarray(keys).reshape(-1)
    d_in = to_device(keys)
    d_out = torch.empty_like(d_in)
    d_idx = torch.empty(keys.size, dtype=torch.int64, device="cuda") if argsort else None
    st = lib.b2s_local_sort_noalloc(_lib.DTYPE_CODE[keys.dtype], d_in.data_ptr(), d_out.data_ptr(),
                                    d_idx.data_ptr() if argsort else None, keys.size, segment, index_offset,
                                    int(ndim_is_1), torch.cuda.current_stream().cuda_stream)
    _lib.check(st, "b2s_local_sort_noalloc")
    # no wait inside the kernels ran out: the status word of the library-held scratch reads 0
    _lib.check(lib.b2s_noalloc_check_status(torch.cuda.current_stream().cuda_stream), "b2s_noalloc_check_status")
    torch.cuda.synchronize()
    return to_host(d_out, keys.dtype), (d_idx.cpu().numpy() if argsort else None)


def test_noalloc_matches_regular_entry_point_twice_in_a_row(cuda_device):
    rng = np.random.default_rng(2024)
    # two different problems back to back: the second call finds the first call's leftovers
    for dtype, n in ((np.float32, 300_000), (np.int64, 200_000)):
        a = random_keys(rng, dtype, n, "full")
        want_k, want_i = cabi_local_sort(a, n, True, index_offset=11, want_keys_too=True)
        got_k, got_i = noalloc_sort(a, n, True, index_offset=11)
        assert_bit_equal(got_k, want_k, f"keys {np.dtype(dtype)}")
        assert np.array_equal(got_i, want_i)
    # and the same problem twice
    a = random_keys(rng, np.uint32, 500_000, "small")
    want_k, _ = cabi_local_sort(a, a.size, False)
    for _ in range(2):
        got_k, _ = noalloc_sort(a, a.size, False)
        assert_bit_equal(got_k, want_k, "repeat")


def test_noalloc_segmented_and_small(cuda_device):
    rng = np.random.default_rng(7)
    a = random_keys(rng, np.float64, 64 * 1000, "small")
    want_k, want_i = cabi_local_sort(a, 1000, True, index_offset=2, ndim_is_1=False, want_keys_too=True)
    got_k, got_i = noalloc_sort(a, 1000, True, index_offset=2, ndim_is_1=False)
    assert_bit_equal(got_k, want_k)
    assert np.array_equal(got_i, want_i)


def test_noalloc_rejects_problems_beyond_its_scratch(cuda_device):
    lib = _lib.lib()
    n = 1 << 24  # needs far more than the 32 MiB the library holds
    fake = ctypes.c_void_p(4096)
    st = lib.b2s_local_sort_noalloc(_lib.DTYPE_CODE[np.dtype(np.int64)], fake, fake, None, n, n, 0, 1, None)
    assert st == 4  # B2S_ERR_WORKSPACE, before anything is launched
    assert lib.b2s_local_sort_noalloc(99, fake, fake, None, 8, 8, 0, 1, None) == 6
