"""The benchmark configurations at their full single-GPU sizes, checked through properties that do
not need a CPU sort of the whole array (permutation, sortedness with NaN last, stability, closed
forms) and cross-checked against torch's own stable sort on the device."""
import numpy as np
import pytest
import torch

import cupynumeric_b200 as num
from cupynumeric_b200 import workloads as w

pytestmark = pytest.mark.gpu


def is_permutation(idx: torch.Tensor) -> bool:
    seen = torch.zeros(idx.numel(), dtype=torch.bool, device=idx.device)
    seen[idx] = True
    return bool(seen.all())


def test_c1_int32_full(cuda_device):
    a = w.c1_int32_uniform()
    got = num.sort(a).to_numpy()
    assert np.array_equal(got, np.sort(a, kind="stable"))


def test_c2_float32_stable_argsort_full(cuda_device):
    a = w.c2_float32_nan_dups()
    arr = num.array(a)
    idx = num.argsort(arr, kind="stable").torch()
    x = arr.torch()
    assert idx.dtype == torch.int64 and idx.numel() == a.size
    assert is_permutation(idx)
    k = x[idx]
    nan = torch.isnan(k)
    n_nan = int(nan.sum())
    assert n_nan == int(np.isnan(a).sum()) and bool(nan[k.numel() - n_nan:].all())   # NaN last
    body, bidx = k[: k.numel() - n_nan], idx[: k.numel() - n_nan]
    assert bool((body[1:] >= body[:-1]).all())                                         # ascending
    ties = body[1:] == body[:-1]
    assert bool((bidx[1:][ties] > bidx[:-1][ties]).all())                              # stable among duplicates
    tail = idx[k.numel() - n_nan:]
    assert bool((tail[1:] > tail[:-1]).all())                                          # stable among NaNs
    assert torch.equal(idx, torch.sort(x, stable=True).indices)


def test_c3_float64_rows_full(cuda_device):
    a = w.c3_float64_rows()
    arr = num.array(a)
    got = num.sort(arr, axis=-1).torch()
    assert bool((got[:, 1:] >= got[:, :-1]).all())
    assert torch.equal(got, torch.sort(arr.torch(), dim=-1).values)
    rows = [0, 1, 4097, 65535]
    assert np.array_equal(got[rows].cpu().numpy(), np.sort(a[rows], axis=-1))


def test_c4_int64_zipf_local(cuda_device):
    a = w.c4_int64_zipf_shard(1 << 24)
    got = num.sort(a).to_numpy()
    assert np.array_equal(got, np.sort(a, kind="stable"))


def test_c5_uint64_nearly_sorted_full(cuda_device):
    n = w.C5_N_PER_GPU
    a = w.c5_uint64_nearly_sorted_shard(n)
    arr = num.array(a)
    idx = num.argsort(arr, kind="stable").torch()
    # the keys are a permutation of 0..n-1: keys[idx[i]] == i
    keys = arr.torch().view(torch.int64)
    assert torch.equal(keys[idx], torch.arange(n, device=idx.device, dtype=torch.int64))
    srt = num.sort(arr).torch().view(torch.int64)
    assert torch.equal(srt, torch.arange(n, device=idx.device, dtype=torch.int64))
