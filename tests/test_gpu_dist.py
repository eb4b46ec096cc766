"""GPU tests of the distributed pieces: the k-way merge on one GPU (all runs resident on it), the
one-rank path of b2s_dist_sort_1d, and - when the box has two GPUs - the full two-rank sort over
NCCL, each against the oracle."""
import ctypes
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from cupynumeric_b200 import _lib
from tests.helpers import assert_bit_equal, random_keys, to_device, to_host

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def kway_merge(runs, payloads=None):
    lib = _lib.lib()
    dtype = runs[0].dtype
    d_runs = [to_device(r) for r in runs]
    d_pay = [torch.from_numpy(p).cuda() for p in payloads] if payloads is not None else None
    n = len(runs)
    total = sum(r.size for r in runs)
    kp = (ctypes.c_void_p * n)(*[t.data_ptr() if t.numel() else None for t in d_runs])
    pp = (ctypes.c_void_p * n)(*[t.data_ptr() if t.numel() else None for t in d_pay]) if d_pay else None
    lens = (ctypes.c_size_t * n)(*[r.size for r in runs])
    need = ctypes.c_size_t()
    _lib.check(lib.b2s_kway_merge_workspace_bytes(total, n, ctypes.byref(need)), "ws")
    ws = torch.empty(max(need.value, 256), dtype=torch.uint8, device="cuda")
    out = torch.empty(max(total, 1), dtype=torch.int64 if payloads is not None else d_runs[0].dtype, device="cuda")
    st = lib.b2s_kway_merge(_lib.DTYPE_CODE[np.dtype(dtype)], n, kp, pp, lens, out.data_ptr(), ws.data_ptr(),
                            ws.numel(), torch.cuda.current_stream().cuda_stream)
    _lib.check(st, "b2s_kway_merge")
    torch.cuda.synchronize()
    out = out[:total]
    return out.cpu().numpy() if payloads is not None else to_host(out, dtype)


@pytest.mark.parametrize("dtype", [np.int64, np.uint64, np.float32, np.int32, np.float64, np.int8, np.float16])
@pytest.mark.parametrize("nruns", [1, 2, 3, 5, 8])
def test_kway_merge_matches_stable_sort_of_concatenation(cuda_device, dtype, nruns):
    rng = np.random.default_rng(nruns * 100 + np.dtype(dtype).itemsize)
    for sizes in ([3000] * nruns, [0] + [1] * (nruns - 1), list(rng.integers(0, 9000, nruns)),
                  [2048 * 3] + [0] * (nruns - 1), [17, 0, 40000][:nruns] if nruns <= 3 else [1, 0, 40000, 5, 0, 7, 2047, 2049][:nruns]):
        flav = "small" if sum(sizes) % 2 else "full"
        runs = [np.sort(random_keys(rng, dtype, int(n), flav), kind="stable") for n in sizes]
        if np.dtype(dtype).kind == "f":   # np.sort puts NaN last, as the merge expects
            pass
        cat = np.concatenate(runs)
        order = np.argsort(cat, kind="stable")
        got = kway_merge(runs)
        assert_bit_equal(got, cat[order], f"merge {np.dtype(dtype)} {sizes}")
        pay = [rng.integers(0, 2**40, r.size).astype(np.int64) for r in runs]
        got_p = kway_merge(runs, pay)
        assert np.array_equal(got_p, np.concatenate(pay)[order]), f"merge payload {np.dtype(dtype)} {sizes}"


def test_kway_merge_heavy_ties_across_runs(cuda_device):
    """Every run holds the same few values: ties must come out in run order."""
    rng = np.random.default_rng(3)
    runs = [np.sort(rng.integers(0, 3, 10000).astype(np.int64)) for _ in range(8)]
    pay = [np.arange(r.size, dtype=np.int64) + i * 1_000_000 for i, r in enumerate(runs)]
    cat = np.concatenate(runs)
    order = np.argsort(cat, kind="stable")
    assert np.array_equal(kway_merge(runs, pay), np.concatenate(pay)[order])


def test_dist_entry_point_single_rank(cuda_device):
    """nranks == 1 through b2s_dist_sort_1d: local sort, result in allocator memory."""
    from cupynumeric_b200._dist import _Pool

    lib = _lib.lib()
    rng = np.random.default_rng(8)
    a = rng.integers(-1000, 1000, 100_000).astype(np.int64)
    d = to_device(a)
    for argsort in (0, 1):
        pool = _Pool()
        out_ptr, out_len = ctypes.c_void_p(), ctypes.c_size_t()
        st = lib.b2s_dist_sort_1d(_lib.DTYPE_CODE[a.dtype], d.data_ptr(), a.size, 1000, argsort, None, 0, 1,
                                  ctypes.cast(pool.alloc_cb, ctypes.c_void_p), ctypes.cast(pool.free_cb, ctypes.c_void_p),
                                  None, None, None, ctypes.byref(out_ptr), ctypes.byref(out_len), None,
                                  torch.cuda.current_stream().cuda_stream)
        _lib.check(st, "dist")
        torch.cuda.synchronize()
        res = pool.adopt(out_ptr.value)[: a.size * 8].view(torch.int64).cpu().numpy()
        assert out_len.value == a.size and len(pool.live) == 0
        want = np.argsort(a, kind="stable") + 1000 if argsort else np.sort(a, kind="stable")
        assert np.array_equal(res, want)


@pytest.mark.parametrize("workload", ["c4", "c5", "f32", "tiny", "mixed", "c64", "empty", "split2d", "search"])
def test_two_rank_sort_over_nccl(cuda_device, workload):
    _two_rank(workload, {})


@pytest.mark.parametrize("workload", ["f32", "mixed", "c4"])
def test_two_rank_sort_nccl_exchange(cuda_device, workload):
    """The same sort with the peer-memory exchange switched off: ncclSend/ncclRecv move the slices."""
    _two_rank(workload, {"B2S_DIST_P2P": "0"})


def test_two_rank_peer_mapping_table_bound(cuda_device):
    """Mappings of other ranks' allocations are closed and reopened when the table is full."""
    _two_rank("recache", {"B2S_PEER_CACHE": "1"})


def _two_rank(workload, extra_env):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", **extra_env)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", "29731", os.path.join(ROOT, "tests", "dist_worker.py"), workload]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "DIST_OK" in r.stdout
