"""The distributed 1-D sort with its ranks as threads of one process on ONE GPU (the thread form of
the collectives table, ``b2s_thread_comm_create``): the whole multi-rank path - samples, weighted
splitters, the partition kernel that writes into the other ranks' receive buffers, the local sort
of what arrived - runs through the C ABI and is compared with the oracle's global stable sort.
Covers 2 to 8 ranks, ragged and empty tiles, heavy duplicates, every key width, both ways of moving
the data, and a rank whose allocator fails (everybody returns an error, nobody waits for ever)."""
import ctypes
import os
import threading

import numpy as np
import pytest
import torch

from cupynumeric_b200 import _lib
from cupynumeric_b200 import workloads as w
from tests.helpers import bits, random_keys, to_device

pytestmark = pytest.mark.gpu


class Pool:
    """Allocator callbacks over torch's caching allocator; ``fail_at`` makes the n-th request fail."""

    def __init__(self, fail_at=None):
        self.live, self.calls, self.fail_at = {}, 0, fail_at
        self.alloc_cb = _lib.ALLOC_FN(self._alloc)
        self.free_cb = _lib.FREE_FN(self._free)

    def _alloc(self, _ctx, nbytes):
        self.calls += 1
        if self.fail_at is not None and self.calls == self.fail_at:
            return None
        t = torch.empty(max(int(nbytes), 256), dtype=torch.uint8, device="cuda")
        self.live[t.data_ptr()] = t
        return t.data_ptr()

    def _free(self, _ctx, ptr):
        self.live.pop(ptr, None)


def run_ranks(shards, argsort, fail=None, timeout=120):
    """Runs one b2s_dist_sort_1d_ops call per rank, each on a thread and a stream of its own.
    Returns [(status, part as numpy or None, global start, pool)] per rank."""
    lib = _lib.lib()
    nranks = len(shards)
    ops = (_lib.CommOps * nranks)()
    _lib.check(lib.b2s_thread_comm_create(nranks, ops), "b2s_thread_comm_create")
    starts = np.cumsum([0] + [s.size for s in shards])
    out = [None] * nranks
    errors = []

    def rank_main(r):
        try:
            torch.cuda.set_device(0)
            stream = torch.cuda.Stream()
            with torch.cuda.stream(stream):
                shard = shards[r]
                d_in = to_device(shard) if shard.size else None
                stream.synchronize()
                pool = Pool(fail_at=fail[1] if fail and fail[0] == r else None)
                out_ptr, out_len, out_start = ctypes.c_void_p(), ctypes.c_size_t(), ctypes.c_int64()
                st = lib.b2s_dist_sort_1d_ops(
                    _lib.DTYPE_CODE[shard.dtype], d_in.data_ptr() if d_in is not None else None, shard.size, int(starts[r]),
                    int(argsort), ctypes.byref(ops[r]), r, nranks, ctypes.cast(pool.alloc_cb, ctypes.c_void_p),
                    ctypes.cast(pool.free_cb, ctypes.c_void_p), None, None, None, ctypes.byref(out_ptr),
                    ctypes.byref(out_len), ctypes.byref(out_start), stream.cuda_stream)
                part = None
                if st == 0:
                    raw = pool.live.pop(out_ptr.value)
                    res_dtype = np.dtype(np.int64) if argsort else shard.dtype
                    part = raw[: out_len.value * res_dtype.itemsize].cpu().numpy().view(res_dtype).copy()
                out[r] = (st, part, int(out_start.value), pool)
        except Exception as e:  # pragma: no cover
            errors.append((r, repr(e)))

    threads = [threading.Thread(target=rank_main, args=(r,), daemon=True) for r in range(nranks)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(timeout)
    alive = [t for t in threads if t.is_alive()]
    assert not alive, "a rank is still waiting for the others"
    assert not errors, errors
    for r in range(nranks):
        lib.b2s_thread_comm_destroy(ctypes.byref(ops[r]))
    return out


def check_against_global_sort(shards, argsort, results, balance=None):
    whole = np.concatenate(shards)
    assert all(st == 0 for st, *_ in results), [st for st, *_ in results]
    got = np.concatenate([p for _, p, _, _ in results])
    order = np.argsort(whole, kind="stable")  # complex keys: NumPy orders by (real, imaginary) as well
    want = order if argsort else whole[order]
    assert got.shape == want.shape
    if argsort:
        assert np.array_equal(got, want), "indices differ from the global stable argsort"
    else:
        assert np.array_equal(bits(got), bits(want)), "values differ from the global stable sort"
    sizes = [p.size for _, p, _, _ in results]
    assert [s for _, _, s, _ in results] == [int(x) for x in np.cumsum([0] + sizes)[:-1]]
    for _, _, _, pool in results:
        assert len(pool.live) == 0, "scratch memory was not handed back"
    if balance is not None and whole.size >= 50_000:
        assert max(sizes) <= balance * whole.size / len(shards) + 64, sizes
    return sizes


@pytest.mark.parametrize("nranks", [2, 3, 4, 8])
@pytest.mark.parametrize("workload", ["c4", "c2", "c5"])
def test_thread_ranks_benchmark_distributions(cuda_device, nranks, workload):
    n = 60_000
    if workload == "c4":
        shards, argsort = [w.c4_int64_zipf_shard(n, r) for r in range(nranks)], False
        shards[-1] = shards[-1][: n // 3]  # ragged
    elif workload == "c2":
        shards, argsort = [w.c2_float32_nan_dups(n, seed=202 + r) for r in range(nranks)], True
    else:
        shards, argsort = [w.c5_uint64_nearly_sorted_shard(n, r, nranks) for r in range(nranks)], True
    res = run_ranks(shards, argsort)
    check_against_global_sort(shards, argsort, res, balance=1.25)


@pytest.mark.parametrize("dtype", [np.int8, np.uint16, np.float16, np.int32, np.float64, np.uint64, np.bool_])
@pytest.mark.parametrize("argsort", [False, True])
def test_thread_ranks_every_key_width(cuda_device, dtype, argsort):
    rng = np.random.default_rng(np.dtype(dtype).itemsize * 7 + int(argsort))
    shards = [random_keys(rng, dtype, m, "full" if i % 2 else "small") for i, m in enumerate((30_000, 12_345, 9_000))]
    res = run_ranks(shards, argsort)
    check_against_global_sort(shards, argsort, res)


@pytest.mark.parametrize("case", ["all_equal", "empty_rank", "only_one_rank", "tiny", "long_and_short", "all_empty"])
def test_thread_ranks_edge_shapes(cuda_device, case):
    rng = np.random.default_rng(11)
    if case == "all_equal":      # one key everywhere: the (rank, position) tie rule must split it evenly
        shards = [np.full(40_000, 7, dtype=np.int64) for _ in range(4)]
    elif case == "empty_rank":
        shards = [rng.integers(-50, 50, 20_000).astype(np.int32), np.empty(0, np.int32), rng.integers(-50, 50, 7).astype(np.int32)]
    elif case == "only_one_rank":
        shards = [np.empty(0, np.int64), np.arange(5000, 0, -1, dtype=np.int64), np.empty(0, np.int64)]
    elif case == "tiny":
        shards = [rng.integers(-5, 5, m).astype(np.int16) for m in (3, 1, 0, 2)]
    elif case == "long_and_short":  # the long tile's elements overflow the short tile's receive buffer
        shards = [rng.integers(0, 1000, 400_000).astype(np.int32), rng.integers(0, 1000, 700).astype(np.int32)]
    else:
        shards = [np.empty(0, np.float32) for _ in range(3)]
    for argsort in (False, True):
        res = run_ranks(shards, argsort)
        sizes = check_against_global_sort(shards, argsort, res)
        if case == "all_equal":
            assert max(sizes) <= 1.1 * 40_000, sizes


@pytest.mark.parametrize("dtype", [np.complex64, np.complex128])
def test_thread_ranks_complex_keys(cuda_device, dtype):
    rng = np.random.default_rng(31)
    shards = [(rng.integers(-30, 30, m) + 1j * rng.integers(-30, 30, m)).astype(dtype) for m in (50_000, 20_000, 33_333)]
    for argsort in (False, True):
        res = run_ranks(shards, argsort)
        check_against_global_sort(shards, argsort, res)


@pytest.mark.parametrize("on", ["0", "1"])
def test_thread_ranks_sender_side_histograms(cuda_device, monkeypatch, on):
    """The senders count the digit histograms of what they send (or not): same results."""
    monkeypatch.setenv("B2S_DIST_SENDER_HIST", on)
    rng = np.random.default_rng(15)
    for dtype, argsort in ((np.float32, True), (np.int64, False), (np.uint16, True), (np.float64, False)):
        if np.dtype(dtype).kind == "f":
            shards = [rng.standard_normal(m).astype(dtype) for m in (50_000, 20_000, 64_123, 9_000)]
            shards[0][::97] = np.nan
        else:
            shards = [rng.integers(0, 1 << 12, m).astype(dtype) for m in (50_000, 20_000, 64_123, 9_000)]  # constant high bytes
        res = run_ranks(shards, argsort)
        check_against_global_sort(shards, argsort, res)


def test_thread_ranks_collective_exchange_branch(cuda_device, monkeypatch):
    """B2S_DIST_P2P=0: the partition is written locally and moved with the table's exchange."""
    monkeypatch.setenv("B2S_DIST_P2P", "0")
    rng = np.random.default_rng(5)
    shards = [rng.standard_normal(m).astype(np.float32) for m in (70_000, 10_000, 40_000)]
    for argsort in (False, True):
        res = run_ranks(shards, argsort)
        check_against_global_sort(shards, argsort, res)


def test_thread_ranks_payload_paths(cuda_device, monkeypatch):
    """Received tiles at or above the single-sort limit (lowered here) and global positions that
    do not fit 32 bits take the position-then-gather path; results stay the global stable argsort."""
    monkeypatch.setenv("B2S_MAX_1D_LOG2", "14")
    rng = np.random.default_rng(6)
    shards = [rng.integers(-1000, 1000, 50_000).astype(np.int32) for _ in range(2)]
    res = run_ranks(shards, True)
    check_against_global_sort(shards, True, res)


@pytest.mark.parametrize("fail", [(1, 1), (0, 2), (2, 3), (1, 4)])
def test_a_rank_whose_allocator_fails_takes_everybody_out_together(cuda_device, fail):
    """Host-side injection: the n-th allocation of one rank returns NULL.  No rank may be left
    waiting in a collective; where the failure is known before the data moves every rank returns
    an error, later only the failing rank does."""
    rng = np.random.default_rng(8)
    shards = [rng.integers(-1000, 1000, 30_000).astype(np.int64) for _ in range(3)]
    res = run_ranks(shards, False, fail=fail, timeout=60)
    statuses = [st for st, *_ in res]
    assert statuses[fail[0]] != 0, statuses
    if fail[1] <= 2:  # control block and receive buffer: known to all before anything is written
        assert all(st != 0 for st in statuses), statuses
    for _, _, _, pool in res:
        assert len(pool.live) == 0, "scratch memory was not handed back"


def run_ranks_nd(tiles, argsort, timeout=120):
    """b2s_dist_sort_nd_ops with thread ranks: ``tiles[r]`` is rank r's (rows, extent_r) slice."""
    lib = _lib.lib()
    nranks = len(tiles)
    ops = (_lib.CommOps * nranks)()
    _lib.check(lib.b2s_thread_comm_create(nranks, ops), "b2s_thread_comm_create")
    out, errors = [None] * nranks, []

    def rank_main(r):
        try:
            torch.cuda.set_device(0)
            stream = torch.cuda.Stream()
            with torch.cuda.stream(stream):
                tile = np.ascontiguousarray(tiles[r])
                d_in = to_device(tile).reshape(tile.shape) if tile.size else None
                d_out = torch.empty(tile.shape, dtype=torch.int64 if argsort else (d_in.dtype if d_in is not None else torch.int32),
                                    device="cuda")
                stream.synchronize()
                pool = Pool()
                st = lib.b2s_dist_sort_nd_ops(_lib.DTYPE_CODE[tile.dtype], d_in.data_ptr() if d_in is not None else None,
                                              d_out.data_ptr() if tile.size else None, int(argsort), tile.shape[0], tile.shape[1],
                                              ctypes.byref(ops[r]), r, nranks, ctypes.cast(pool.alloc_cb, ctypes.c_void_p),
                                              ctypes.cast(pool.free_cb, ctypes.c_void_p), None, None, None, stream.cuda_stream)
                res = d_out.cpu().numpy() if argsort else d_out.cpu().numpy().view(tile.dtype)
                out[r] = (st, res, pool)
        except Exception as e:  # pragma: no cover
            errors.append((r, repr(e)))

    threads = [threading.Thread(target=rank_main, args=(r,), daemon=True) for r in range(nranks)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(timeout)
    assert not [t for t in threads if t.is_alive()], "a rank is still waiting for the others"
    assert not errors, errors
    for r in range(nranks):
        lib.b2s_thread_comm_destroy(ctypes.byref(ops[r]))
    return out


@pytest.mark.parametrize("dtype", [np.int32, np.float64, np.int16, np.complex64])
@pytest.mark.parametrize("shape", [(8, (100, 37, 250)), (300, (7, 0, 5, 9)), (5, (3000, 9000)), (2, (10, 10, 10)), (64, (4096, 4096))])
def test_split_axis_rows_all_at_once(cuda_device, dtype, shape):
    """Rows whose sort axis is split over the ranks (ragged extents, an empty slice, fewer rows than
    ranks, rows too long for the on-chip sort): every rank ends up with its own extent of every
    sorted row, values and stable argsort positions."""
    rows, extents = shape
    rng = np.random.default_rng(rows + len(extents))
    if np.dtype(dtype).kind == "c":
        whole = (rng.integers(-9, 9, (rows, sum(extents))) + 1j * rng.integers(-9, 9, (rows, sum(extents)))).astype(dtype)
    else:
        whole = rng.integers(-50, 50, (rows, sum(extents))).astype(dtype)
    cuts = np.cumsum((0,) + tuple(extents))
    tiles = [whole[:, cuts[r]:cuts[r + 1]] for r in range(len(extents))]
    for argsort in (False, True):
        res = run_ranks_nd(tiles, argsort)
        assert all(st == 0 for st, _, _ in res), [st for st, _, _ in res]
        got = np.concatenate([r for _, r, _ in res], axis=1)
        want = np.argsort(whole, axis=1, kind="stable") if argsort else np.sort(whole, axis=1, kind="stable")
        assert np.array_equal(got, want)
        assert all(len(pool.live) == 0 for _, _, pool in res)
