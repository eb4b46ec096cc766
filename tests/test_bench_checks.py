"""The benchmark's own result checks, exercised on CPU tensors: they accept the true result and
reject results with one wrong element, an unstable tie, a missing element or a wrong multiset."""
import numpy as np
import pytest
import torch

import bench


def _np_order_keys(a):
    """NumPy's stable argsort defines the total order the checker must reproduce."""
    return np.argsort(a, kind="stable")


@pytest.mark.parametrize("dtype", [np.int32, np.int64, np.uint64, np.float32, np.float64, np.float16, np.uint32])
def test_ordered_view_reproduces_the_sort_order(dtype):
    rng = np.random.default_rng(5)
    if np.dtype(dtype).kind == "f":
        a = rng.standard_normal(4000).astype(dtype)
        a[::97] = np.nan
        a[::89] = -0.0
        a[::83] = 0.0
        a[::79] = np.inf
        a[::73] = -np.inf
    else:
        info = np.iinfo(dtype)
        a = rng.integers(info.min, info.max, 4000, dtype=dtype, endpoint=True)
    t = torch.from_numpy(a.view({np.dtype(np.uint64): np.int64, np.dtype(np.uint32): np.int32}.get(np.dtype(dtype), dtype)))
    if dtype == np.uint64:
        t = t.view(torch.uint64)
    if dtype == np.uint32:
        t = t.view(torch.uint32)
    o = bench.ordered_i64(t).numpy()
    assert np.array_equal(np.argsort(o, kind="stable"), _np_order_keys(a))


def _c(name):
    return bench.CONFIGS[name]


def test_full_check_accepts_the_sort_and_rejects_corruptions():
    rng = np.random.default_rng(1)
    a = rng.integers(-50, 50, 10_000).astype(np.int64)
    tile = torch.from_numpy(a)
    good = torch.from_numpy(np.sort(a, kind="stable"))
    ok, detail = bench.check_full("c4", tile, good, 0, 0, 1, None)
    assert ok, detail
    bad = good.clone()
    bad[17], bad[18] = good[9000], good[18]
    assert not bench.check_full("c4", tile, bad, 0, 0, 1, None)[0]          # not sorted, wrong multiset
    bad = good.clone()
    bad[-1] = bad[-1] + 1                                                   # still sorted, wrong multiset
    assert not bench.check_full("c4", tile, bad, 0, 0, 1, None)[0]
    assert not bench.check_full("c4", tile, good[:-1], 0, 0, 1, None)[0]    # an element is missing


def test_full_check_of_an_argsort_pins_stability():
    rng = np.random.default_rng(2)
    a = rng.standard_normal(5000).astype(np.float32)
    a[::7] = a[3]
    a[::11] = np.nan
    tile = torch.from_numpy(a)
    good = torch.from_numpy(np.argsort(a, kind="stable"))
    ok, detail = bench.check_full("c2", tile, good, 0, 0, 1, None)
    assert ok, detail
    # swap two indices of one tie: still sorts the keys, no longer stable
    g = good.numpy().copy()
    ties = np.flatnonzero(a[g][1:] == a[g][:-1])
    j = int(ties[0])
    g[j], g[j + 1] = g[j + 1], g[j]
    assert not bench.check_full("c2", tile, torch.from_numpy(g), 0, 0, 1, None)[0]
    g = good.numpy().copy()
    g[5] = g[6]                                                             # not a permutation
    assert not bench.check_full("c2", tile, torch.from_numpy(g), 0, 0, 1, None)[0]


def test_full_check_of_row_sorts():
    rng = np.random.default_rng(3)
    a = rng.random((16, 4096))
    good = np.sort(a, axis=1)
    assert bench.check_full("c3", torch.from_numpy(a), torch.from_numpy(good), 0, 0, 1, None)[0]
    bad = good.copy()
    bad[3, 10] = bad[3, 11]
    assert not bench.check_full("c3", torch.from_numpy(a), torch.from_numpy(bad), 0, 0, 1, None)[0]


def test_reference_arm_prints_one_line(capsys, monkeypatch):
    import json
    import sys

    monkeypatch.setattr(sys, "argv", ["bench.py", "--impl", "reference", "--workload", "c1", "--scale-log2", "16",
                                      "--steps", "2", "--warmup", "1"])
    monkeypatch.setenv("OMP_NUM_THREADS", "1")   # what torch.distributed.run exports to its children
    bench.main()
    line = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["cpu_baseline"]["cores"] == bench.host_threads()
    assert line["steps"] == 2 and line["e2e"]["h2d_bytes_per_step"] == 0
